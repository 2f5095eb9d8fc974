// Stand-in for llvm::StringRef: a string view with the .str() the reference's builders call.
#pragma once

#include <string>
#include <string_view>

namespace llvm {

class StringRef : public std::string_view {
 public:
  using std::string_view::string_view;
  StringRef(const std::string& s) : std::string_view(s) {}   // NOLINT: implicit by design
  StringRef(const char* s) : std::string_view(s) {}          // NOLINT
  std::string str() const { return std::string(*this); }
};

}  // namespace llvm
