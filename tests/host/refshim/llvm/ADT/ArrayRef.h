// Stand-in for llvm::ArrayRef (a non-owning view of contiguous elements), as far as the reference's
// network builders use it.
#pragma once

#include <cstddef>
#include <initializer_list>
#include <vector>

namespace llvm {

template <typename T>
class ArrayRef {
 public:
  ArrayRef() = default;
  ArrayRef(const T* data, size_t size) : data_(data), size_(size) {}
  ArrayRef(const std::vector<T>& v) : data_(v.data()), size_(v.size()) {}          // NOLINT: implicit by design
  ArrayRef(const std::initializer_list<T>& l) : data_(l.begin()), size_(l.size()) {}  // NOLINT
  template <typename C, typename = decltype(std::declval<const C&>().data()), typename = decltype(std::declval<const C&>().size())>
  ArrayRef(const C& c) : data_(c.data()), size_(c.size()) {}                          // NOLINT
  const T& operator[](size_t i) const { return data_[i]; }
  const T* begin() const { return data_; }
  const T* end() const { return data_ + size_; }
  size_t size() const { return size_; }
  bool empty() const { return size_ == 0; }
  std::vector<T> vec() const { return std::vector<T>(data_, data_ + size_); }

 private:
  const T* data_ = nullptr;
  size_t size_ = 0;
};

}  // namespace llvm
