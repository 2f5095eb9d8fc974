// Stand-in for llvm::SmallVector: a std::vector (the inline capacity is a performance hint only).
#pragma once

#include <initializer_list>
#include <vector>

namespace llvm {

template <typename T, unsigned N = 4>
class SmallVector : public std::vector<T> {
 public:
  using std::vector<T>::vector;
  SmallVector(std::initializer_list<T> l) : std::vector<T>(l) {}
};

}  // namespace llvm
