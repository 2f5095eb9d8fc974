// Stand-in for llvm/Support/FormatVariadic.h as far as the reference's command-line programs use it:
// llvm::formatv("...{0}...{1}...", a, b) with plain positional placeholders, convertible to std::string.
#pragma once

#include <sstream>
#include <string>
#include <vector>

namespace llvm {

class formatv_object {
 public:
  formatv_object(const char* fmt, std::vector<std::string> args) {
    const std::string f(fmt);
    for (size_t i = 0; i < f.size(); ++i) {
      if (f[i] == '{') {
        const size_t close = f.find('}', i);
        if (close != std::string::npos) {
          const size_t index = static_cast<size_t>(std::stoul(f.substr(i + 1, close - i - 1)));
          if (index < args.size()) text_ += args[index];
          i = close;
          continue;
        }
      }
      text_ += f[i];
    }
  }
  std::string str() const { return text_; }
  operator std::string() const { return text_; }

 private:
  std::string text_;
};

template <typename... Ts>
formatv_object formatv(const char* fmt, const Ts&... values) {
  std::vector<std::string> args;
  auto add = [&](const auto& v) {
    std::ostringstream os;
    os << v;
    args.push_back(os.str());
  };
  (add(values), ...);
  return formatv_object(fmt, std::move(args));
}

}  // namespace llvm
