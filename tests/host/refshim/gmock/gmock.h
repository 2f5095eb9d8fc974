// Stand-in: the reference's test sources include gmock for matchers their fixture uses; the fixture
// here (plaidml/testenv.h of this directory) compares by itself.
#pragma once
#include "gtest/gtest.h"

#include <sstream>
#include <string>
#include <tuple>

// The handful of matchers the reference's EDSL tests use with EXPECT_THAT.
namespace testing {

struct HasSubstrMatcher {
  std::string needle;
  template <typename T>
  bool Matches(const T& v) const { return std::string(v).find(needle) != std::string::npos; }
};
inline HasSubstrMatcher HasSubstr(const std::string& s) { return {s}; }

template <typename V>
struct EqMatcher {
  V want;
  template <typename T>
  bool Matches(const T& v) const { return v == want; }
};
template <typename V>
EqMatcher<V> Eq(const V& v) { return {v}; }

template <typename C>
struct ContainerEqMatcher {
  C want;
  template <typename T>
  bool Matches(const T& v) const { return v == want; }
};
template <typename C>
ContainerEqMatcher<C> ContainerEq(const C& c) { return {c}; }

template <typename... M>
struct AnyOfMatcher {
  std::tuple<M...> ms;
  template <typename T>
  bool Matches(const T& v) const {
    return std::apply([&](const auto&... m) { return (m.Matches(v) || ...); }, ms);
  }
};
template <typename... M>
AnyOfMatcher<M...> AnyOf(const M&... m) { return {std::make_tuple(m...)}; }

}  // namespace testing

#define EXPECT_THAT(value, matcher)                                              \
  do {                                                                           \
    if (!(matcher).Matches(value)) ::testing::fail("EXPECT_THAT(" #value ", " #matcher ")"); \
  } while (0)
