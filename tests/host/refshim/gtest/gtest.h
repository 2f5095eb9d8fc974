// A few lines standing in for googletest, so that test sources of the reference checkout compile and run
// unmodified against libplaidml.so: a registry of TEST_F bodies and a failure counter.  Only what those
// sources use is here (fixtures and TEST_F; their checks go through the fixture in plaidml/testenv.h).
#pragma once

#include <functional>
#include <iostream>
#include <limits>   // (googletest's own header brings it in; one of the reference's examples relies on that)
#include <string>
#include <vector>

namespace testing {

class Test {
 public:
  virtual ~Test() = default;
  virtual void SetUp() {}
  virtual void TearDown() {}
  virtual void TestBody() = 0;
};

struct Registry {
  struct Entry {
    std::string name;
    std::function<Test*()> make;
  };
  static std::vector<Entry>& tests() {
    static std::vector<Entry> t;
    return t;
  }
  static int& failures() {
    static int n = 0;
    return n;
  }
  static int add(const std::string& name, std::function<Test*()> make) {
    tests().push_back({name, std::move(make)});
    return 0;
  }
};

inline void fail(const std::string& what) {
  ++Registry::failures();
  std::cout << "  FAILED: " << what << std::endl;
}

}  // namespace testing

#define TEST_F(fixture, name)                                                                        \
  class fixture##_##name##_Test : public fixture {                                                   \
   public:                                                                                           \
    void TestBody() override;                                                                        \
  };                                                                                                 \
  static int fixture##_##name##_registered =                                                         \
      ::testing::Registry::add(#fixture "." #name, [] { return new fixture##_##name##_Test(); });    \
  void fixture##_##name##_Test::TestBody()

#define EXPECT_ANY_THROW(statement)                                                    \
  do {                                                                                 \
    bool pmlb_threw = false;                                                           \
    try { statement; } catch (...) { pmlb_threw = true; }                              \
    if (!pmlb_threw) ::testing::fail("expected an exception: " #statement);            \
  } while (0)

#define EXPECT_NO_THROW(statement)                                                     \
  do {                                                                                 \
    try { statement; } catch (const std::exception& e) {                               \
      ::testing::fail(std::string("unexpected exception: ") + e.what());               \
    } catch (...) { ::testing::fail("unexpected exception: " #statement); }            \
  } while (0)

// Value-parameterised tests (TEST_P / INSTANTIATE_TEST_CASE_P with ::testing::ValuesIn), as far as the reference's
// op tests use them: every TEST_P body of a fixture runs once per value.
namespace testing {

template <typename T>
class WithParamInterface {
 public:
  using ParamType = T;
  static const T& GetParam() { return *current(); }
  static const T*& current() {
    static const T* p = nullptr;
    return p;
  }
};

template <typename Fixture>
struct ParamBodies {
  struct Body {
    std::string name;
    std::function<Test*()> make;
  };
  static std::vector<Body>& list() {
    static std::vector<Body> l;
    return l;
  }
  static int add(const std::string& name, std::function<Test*()> make) {
    list().push_back({name, std::move(make)});
    return 0;
  }
};

template <typename Container>
std::vector<typename Container::value_type> ValuesIn(const Container& c) {
  return std::vector<typename Container::value_type>(c.begin(), c.end());
}
template <typename T, size_t N>
std::vector<T> ValuesIn(const T (&array)[N]) {
  return std::vector<T>(array, array + N);
}

template <typename Fixture, typename T>
int instantiate(const std::string& prefix, const std::string& fixture, const std::vector<T>& values) {
  auto* stored = new std::vector<T>(values);   // lives as long as the registry
  for (size_t i = 0; i < stored->size(); ++i) {
    for (const auto& body : ParamBodies<Fixture>::list()) {
      auto make = body.make;
      Registry::add(prefix + "/" + fixture + "." + body.name + "/" + std::to_string(i), [stored, i, make] {
        WithParamInterface<T>::current() = &(*stored)[i];
        return make();
      });
    }
  }
  return 0;
}

}  // namespace testing

#define TEST_P(fixture, name)                                                                          \
  class fixture##_##name##_Test : public fixture {                                                     \
   public:                                                                                             \
    void TestBody() override;                                                                          \
  };                                                                                                   \
  static int fixture##_##name##_registered =                                                           \
      ::testing::ParamBodies<fixture>::add(#name, [] { return new fixture##_##name##_Test(); });       \
  void fixture##_##name##_Test::TestBody()

#define INSTANTIATE_TEST_CASE_P(prefix, fixture, generator) \
  static int prefix##_##fixture##_instantiated = ::testing::instantiate<fixture>(#prefix, #fixture, generator)
#define INSTANTIATE_TEST_SUITE_P(prefix, fixture, generator) INSTANTIATE_TEST_CASE_P(prefix, fixture, generator)
