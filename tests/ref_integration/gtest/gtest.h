// A minimal stand-in for <gtest/gtest.h>: just enough of the GoogleTest interface
// to compile and run the reference project's integration tests
// (tests/integration/operations/*.cpp: TEST_F fixtures, EXPECT_FLOAT_EQ, GTEST_SKIP)
// where GoogleTest itself is not installed.  Test infrastructure only.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

namespace testing {

class Test {
public:
  virtual ~Test() = default;
  virtual void SetUp() {}
  virtual void TearDown() {}
  virtual void TestBody() = 0;
  bool skipped = false;
};

class Message {
public:
  template <typename T> Message& operator<<(const T& v) {
    mStream << v;
    return *this;
  }
  std::string str() const { return mStream.str(); }

private:
  std::ostringstream mStream;
};

namespace internal {

struct Entry {
  const char* suite;
  const char* name;
  Test* (*make)();
};
inline std::vector<Entry>& registry() {
  static std::vector<Entry> r;
  return r;
}
inline int& failures() {
  static int n = 0;
  return n;
}
struct Registrar {
  Registrar(const char* suite, const char* name, Test* (*make)()) { registry().push_back({suite, name, make}); }
};

// `return SkipHelper(this) = Message() << "why";` marks the running test as skipped.
struct SkipHelper {
  explicit SkipHelper(Test* t) : test(t) {}
  void operator=(const Message& m) const {
    test->skipped = true;
    std::printf("[  SKIPPED ] %s\n", m.str().c_str());
  }
  Test* test;
};

// GoogleTest's float comparison: equal within 4 units in the last place; NaN never equal.
inline bool almostEqual(float a, float b) {
  if (std::isnan(a) || std::isnan(b)) return false;
  auto biased = [](float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? (~u + 1) : (u | 0x80000000u);
  };
  uint32_t x = biased(a), y = biased(b);
  return (x > y ? x - y : y - x) <= 4;
}
inline void expectFloatEq(const char* ea, const char* eb, float a, float b, const char* file, int line) {
  if (almostEqual(a, b)) return;
  ++failures();
  std::printf("%s:%d: Failure\nExpected equality of these values:\n  %s\n    Which is: %.9g\n  %s\n    Which is: %.9g\n",
              file, line, ea, a, eb, b);
}

}  // namespace internal
}  // namespace testing

#define TEST_F(fixture, name)                                                              \
  class fixture##_##name##_Test : public fixture {                                         \
  public:                                                                                  \
    void TestBody() override;                                                              \
  };                                                                                       \
  static ::testing::internal::Registrar fixture##_##name##_registrar(                      \
      #fixture, #name, []() -> ::testing::Test* { return new fixture##_##name##_Test; });  \
  void fixture##_##name##_Test::TestBody()

#define EXPECT_FLOAT_EQ(a, b) \
  ::testing::internal::expectFloatEq(#a, #b, static_cast<float>(a), static_cast<float>(b), __FILE__, __LINE__)

#define GTEST_SKIP() return ::testing::internal::SkipHelper(this) = ::testing::Message()
