// A few lines standing in for googletest, so that test sources of the reference checkout compile and run
// unmodified against libplaidml.so: a registry of TEST_F bodies and a failure counter.  Only what those
// sources use is here (fixtures and TEST_F; their checks go through the fixture in plaidml/testenv.h).
#pragma once

#include <functional>
#include <iostream>
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
