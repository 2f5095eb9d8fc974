// Core data model: element types, shapes, pinned host buffers, settings.
#include "pml_core.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace pml {

size_t dtypeBytes(DType t) {
  switch (t) {
    case DType::i1:
    case DType::si8:
    case DType::ui8: return 1;
    case DType::si16:
    case DType::ui16:
    case DType::f16:
    case DType::bf16: return 2;
    case DType::six:
    case DType::uix:
    case DType::fx:
    case DType::si32:
    case DType::ui32:
    case DType::f32: return 4;
    case DType::si64:
    case DType::ui64:
    case DType::f64: return 8;
    default: return 0;
  }
}

const char* dtypeName(DType t) {
  switch (t) {
    case DType::six: return "six";
    case DType::uix: return "uix";
    case DType::fx: return "fx";
    case DType::i1: return "i1";
    case DType::si8: return "si8";
    case DType::ui8: return "ui8";
    case DType::si16: return "si16";
    case DType::ui16: return "ui16";
    case DType::si32: return "si32";
    case DType::ui32: return "ui32";
    case DType::si64: return "si64";
    case DType::ui64: return "ui64";
    case DType::f16: return "f16";
    case DType::bf16: return "bf16";
    case DType::f32: return "f32";
    case DType::f64: return "f64";
    default: return "invalid";
  }
}

bool isFloat(DType t) {
  return t == DType::f16 || t == DType::bf16 || t == DType::f32 || t == DType::f64 || t == DType::fx;
}

bool isSignedInt(DType t) {
  return t == DType::si8 || t == DType::si16 || t == DType::si32 || t == DType::si64 || t == DType::six;
}

bool isAmbiguous(DType t) { return t == DType::six || t == DType::uix || t == DType::fx; }

int typeScore(DType t) {
  if (t == DType::bf16) return 27;              // between f16 (26) and f32 (28)
  return 2 * static_cast<int>(t);
}

DType promote(DType a, DType b) { return typeScore(a) > typeScore(b) ? a : b; }

DType fromFfi(plaidml_datatype dt) {
  if (dt < PLAIDML_DATA_INVALID || dt > PLAIDML_DATA_BFLOAT16) throw std::runtime_error("Invalid plaidml_datatype");
  return static_cast<DType>(dt);
}

plaidml_datatype toFfi(DType dt) { return static_cast<plaidml_datatype>(dt); }

int64_t TensorShape::elements() const {
  int64_t n = 1;
  for (int64_t s : sizes) n *= s;
  return n;
}

size_t TensorShape::byteSize() const {
  // Strided shapes occupy the span their largest element reaches (pmlc/util/shape.cc:60-75).
  if (strides.empty()) return static_cast<size_t>(elements()) * dtypeBytes(dtype);
  int64_t span = 1;
  for (size_t i = 0; i < sizes.size(); ++i) {
    if (sizes[i] == 0) return 0;
    span += (sizes[i] - 1) * strides[i];
  }
  return static_cast<size_t>(span) * dtypeBytes(dtype);
}

std::vector<int64_t> TensorShape::denseStrides() const {
  std::vector<int64_t> st(sizes.size());
  int64_t s = 1;
  for (size_t i = sizes.size(); i-- > 0;) {
    st[i] = s;
    s *= sizes[i];
  }
  return st;
}

bool TensorShape::isDense() const { return strides.empty() || strides == denseStrides(); }

std::string TensorShape::str() const {
  std::ostringstream os;
  os << "tensor<";
  for (int64_t s : sizes) os << s << "x";
  os << dtypeName(dtype) << ">";
  return os.str();
}

// The spelling plaidml_shape_repr returns in the reference (pmlc/util/shape.cc:69-91): sizes joined by 'x'
// (a zero size prints as '?'), the element type, then the strides only when the shape carries them.
std::string TensorShape::repr() const {
  std::ostringstream os;
  for (int64_t s : sizes) {
    if (s) os << s; else os << '?';
    os << 'x';
  }
  os << dtypeName(dtype);
  if (!strides.empty()) {
    os << ", [";
    for (size_t i = 0; i < strides.size(); ++i) os << (i ? "x" : "") << strides[i];
    os << ']';
  }
  return os.str();
}

bool TensorShape::operator==(const TensorShape& rhs) const {
  return dtype == rhs.dtype && sizes == rhs.sizes && effectiveStrides() == rhs.effectiveStrides();
}

// ------------------------------------------------------------------ buffers

namespace {
bool cudaUsable() {
  static int state = -1;
  if (state < 0) {
    int n = 0;
    state = (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? 1 : 0;
    if (!state) cudaGetLastError();
  }
  return state == 1;
}
}  // namespace

BufferPtr Buffer::allocate(const TensorShape& shape) {
  std::shared_ptr<Buffer> buf(new Buffer());
  buf->shape_ = shape;
  buf->size_ = shape.byteSize();
  buf->owned_ = true;
  const size_t bytes = buf->size_ ? buf->size_ : 1;
  if (cudaUsable()) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) == cudaSuccess) {
      buf->data_ = static_cast<char*>(p);
      buf->pinned_ = true;
    } else {
      cudaGetLastError();
    }
  }
  if (!buf->data_) {
    buf->data_ = static_cast<char*>(std::malloc(bytes));
    if (!buf->data_) throw std::bad_alloc();
  }
  std::memset(buf->data_, 0, bytes);
  return buf;
}

BufferPtr Buffer::adopt(const TensorShape& shape, char* data, size_t size) {
  if (size < shape.byteSize()) throw std::runtime_error("Adopted buffer is smaller than its shape");
  std::shared_ptr<Buffer> buf(new Buffer());
  buf->shape_ = shape;
  buf->size_ = size;
  buf->data_ = data;
  return buf;
}

Buffer::~Buffer() {
  if (owned_ && data_) {
    if (pinned_) {
      cudaFreeHost(data_);
    } else {
      std::free(data_);
    }
  }
}

// ------------------------------------------------------------------ settings

std::string getEnv(const std::string& key, const std::string& fallback) {
  const char* v = std::getenv(key.c_str());
  return v ? std::string(v) : fallback;
}

namespace {
std::string settingsPath() {
  std::string p = getEnv("PLAIDML_SETTINGS");
  if (!p.empty()) return p;
  const std::string home = getEnv("HOME");
  return home.empty() ? std::string(".plaidml2") : home + "/.plaidml2";
}
}  // namespace

Settings::Settings() { load(); }

Settings& Settings::instance() {
  static Settings s;
  return s;
}

void Settings::load() {
  kvs_.clear();
  std::ifstream in(settingsPath());
  std::string line;
  while (std::getline(in, line)) {
    const size_t eq = line.find('=');
    if (eq == std::string::npos) continue;
    const std::string key = line.substr(0, eq), value = line.substr(eq + 1);
    bool found = false;
    for (auto& kv : kvs_) {
      if (kv.first == key) {
        kv.second = value;
        found = true;
      }
    }
    if (!found) kvs_.emplace_back(key, value);
    // the environment wins over the file; export only what the environment lacks
    if (std::getenv(key.c_str()) == nullptr) setenv(key.c_str(), value.c_str(), 1);
  }
}

void Settings::save() {
  std::ofstream out(settingsPath());
  for (const auto& kv : kvs_) out << kv.first << "=" << kv.second << "\n";
}

std::string Settings::get(const std::string& key) {
  const char* env = std::getenv(key.c_str());
  if (env) return env;
  for (const auto& kv : kvs_) {
    if (kv.first == key) return kv.second;
  }
  throw std::runtime_error("Unknown setting: " + key);
}

std::string Settings::getOr(const std::string& key, const std::string& fallback) {
  const char* env = std::getenv(key.c_str());
  if (env) return env;
  for (const auto& kv : kvs_) {
    if (kv.first == key) return kv.second;
  }
  return fallback;
}

void Settings::set(const std::string& key, const std::string& value) {
  bool found = false;
  for (auto& kv : kvs_) {
    if (kv.first == key) {
      kv.second = value;
      found = true;
    }
  }
  if (!found) kvs_.emplace_back(key, value);
  setenv(key.c_str(), value.c_str(), 1);
}

std::vector<std::pair<std::string, std::string>> Settings::all() {
  auto out = kvs_;
  for (auto& kv : out) {
    const char* env = std::getenv(kv.first.c_str());
    if (env) kv.second = env;
  }
  return out;
}

}  // namespace pml
