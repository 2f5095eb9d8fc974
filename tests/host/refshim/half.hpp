// Stand-in for the third-party half.hpp the reference's tests include (half_float::half): IEEE binary16 storage
// with conversion from and to float, which is all those tests use (filling inputs, holding expected values).
#pragma once

#include <cstdint>
#include <cstring>

namespace half_float {

class half {
 public:
  half() = default;
  half(float f) : bits_(fromFloat(f)) {}  // NOLINT
  half(double d) : bits_(fromFloat(static_cast<float>(d))) {}  // NOLINT
  half(int i) : bits_(fromFloat(static_cast<float>(i))) {}  // NOLINT
  operator float() const { return toFloat(bits_); }
  bool operator==(const half& o) const { return static_cast<float>(*this) == static_cast<float>(o); }
  bool operator!=(const half& o) const { return !(*this == o); }

 private:
  static uint16_t fromFloat(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0u));   // inf / nan
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);                                           // overflow
    if (exp <= 0) {
      if (exp < -10) return static_cast<uint16_t>(sign);                                                   // underflow to zero
      man |= 0x800000u;
      const int shift = 14 - exp;
      uint32_t h = man >> shift;
      const uint32_t rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
      if (rem > halfway || (rem == halfway && (h & 1u))) ++h;
      return static_cast<uint16_t>(sign | h);
    }
    uint32_t h = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;   // round to nearest even (may carry into the exponent)
    return static_cast<uint16_t>(sign | h);
  }
  static float toFloat(uint16_t h) {
    const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, x;
    if (exp == 0) {
      if (man == 0) {
        x = sign;
      } else {
        int e = -1;
        do {
          ++e;
          man <<= 1;
        } while (!(man & 0x400u));
        x = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man & 0x3ffu) << 13;
      }
    } else if (exp == 31) {
      x = sign | 0x7f800000u | man << 13;
    } else {
      x = sign | (exp + 127 - 15) << 23 | man << 13;
    }
    float f;
    std::memcpy(&f, &x, 4);
    return f;
  }
  uint16_t bits_ = 0;
};

}  // namespace half_float
