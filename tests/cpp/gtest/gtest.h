// Minimal single-header stand-in for the parts of GoogleTest that micrograd's
// test suite uses (TEST, EXPECT_NEAR and a gtest_main-style entry point), plus a
// few more checks for this repository's own C++ tests.  GoogleTest itself is
// fetched from the network by the reference's build and is not available
// offline; with this header on the include path, `#include <gtest/gtest.h>`
// resolves here and a test file written for GoogleTest compiles unchanged.
//
// One translation unit per test binary: the header defines main() unless
// MG_GTEST_NO_MAIN is defined before inclusion.
#pragma once

#include <cmath>
#include <cstdio>
#include <exception>
#include <functional>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace testing {

struct TestCase {
  std::string suite;
  std::string name;
  std::function<void()> body;
};

inline std::vector<TestCase> &registry() {
  static std::vector<TestCase> r;
  return r;
}

inline int &current_failures() {
  static int f = 0;
  return f;
}

struct Registrar {
  Registrar(const char *suite, const char *name, std::function<void()> body) {
    registry().push_back({suite, name, std::move(body)});
  }
};

// Collects a streamed user message and prints the failure when destroyed.
class Failure {
public:
  Failure(const char *file, int line, const std::string &what) {
    os_ << file << ":" << line << ": Failure\n" << what;
  }
  ~Failure() {
    std::cout << os_.str() << std::endl;
    current_failures()++;
  }
  template <class T> Failure &operator<<(const T &v) {
    os_ << "\n" << v;
    return *this;
  }

private:
  std::ostringstream os_;
};

// Lets `return Voidify() & Failure(...)` appear in a void function (ASSERT_*).
struct Voidify {
  void operator&(const Failure &) {}
};

template <class A, class B, class T>
inline std::string near_msg(const char *ea, const char *eb, const A &a, const B &b, const T &tol) {
  std::ostringstream os;
  os.precision(17);
  os << "The difference between " << ea << " and " << eb << " is "
     << std::fabs(static_cast<double>(a) - static_cast<double>(b)) << ", which exceeds " << tol
     << "\n  " << ea << " evaluates to " << a << "\n  " << eb << " evaluates to " << b;
  return os.str();
}

template <class A, class B>
inline std::string cmp_msg(const char *op, const char *ea, const char *eb, const A &a, const B &b) {
  std::ostringstream os;
  os.precision(17);
  os << "Expected: (" << ea << ") " << op << " (" << eb << "), actual: " << a << " vs " << b;
  return os.str();
}

inline int run_all(int argc, char **argv) {
  std::string filter;
  for (int i = 1; i < argc; i++) {
    std::string a = argv[i];
    const std::string key = "--gtest_filter=";
    if (a.rfind(key, 0) == 0) {
      filter = a.substr(key.size());
    }
  }
  int failed = 0, ran = 0;
  for (auto &t : registry()) {
    std::string full = t.suite + "." + t.name;
    if (!filter.empty() && full.find(filter) == std::string::npos) {
      continue;
    }
    std::cout << "[ RUN      ] " << full << std::endl;
    current_failures() = 0;
    try {
      t.body();
    } catch (const std::exception &e) {
      std::cout << "unexpected exception: " << e.what() << std::endl;
      current_failures()++;
    } catch (...) {
      std::cout << "unexpected non-standard exception" << std::endl;
      current_failures()++;
    }
    ran++;
    if (current_failures() == 0) {
      std::cout << "[       OK ] " << full << std::endl;
    } else {
      std::cout << "[  FAILED  ] " << full << std::endl;
      failed++;
    }
  }
  std::cout << "[==========] " << ran << " tests ran." << std::endl;
  std::cout << "[  PASSED  ] " << (ran - failed) << " tests." << std::endl;
  if (failed) {
    std::cout << "[  FAILED  ] " << failed << " tests." << std::endl;
  }
  return failed == 0 ? 0 : 1;
}

} // namespace testing

#define MG_GTEST_NAME(suite, name) suite##_##name##_Test

#define TEST(suite, name)                                                                          \
  static void MG_GTEST_NAME(suite, name)();                                                        \
  static ::testing::Registrar MG_GTEST_NAME(suite, name##_reg)(#suite, #name,                      \
                                                               MG_GTEST_NAME(suite, name));        \
  static void MG_GTEST_NAME(suite, name)()

#define MG_GTEST_CHECK(cond, msg)                                                                  \
  if (cond)                                                                                        \
    ;                                                                                              \
  else                                                                                             \
    ::testing::Failure(__FILE__, __LINE__, msg)

#define MG_GTEST_CHECK_FATAL(cond, msg)                                                            \
  if (cond)                                                                                        \
    ;                                                                                              \
  else                                                                                             \
    return ::testing::Voidify() & ::testing::Failure(__FILE__, __LINE__, msg)

#define EXPECT_NEAR(a, b, tol)                                                                     \
  MG_GTEST_CHECK(std::fabs(static_cast<double>(a) - static_cast<double>(b)) <=                     \
                     static_cast<double>(tol),                                                     \
                 ::testing::near_msg(#a, #b, (a), (b), (tol)))
#define ASSERT_NEAR(a, b, tol)                                                                     \
  MG_GTEST_CHECK_FATAL(std::fabs(static_cast<double>(a) - static_cast<double>(b)) <=               \
                           static_cast<double>(tol),                                               \
                       ::testing::near_msg(#a, #b, (a), (b), (tol)))

#define EXPECT_EQ(a, b) MG_GTEST_CHECK((a) == (b), ::testing::cmp_msg("==", #a, #b, (a), (b)))
#define ASSERT_EQ(a, b) MG_GTEST_CHECK_FATAL((a) == (b), ::testing::cmp_msg("==", #a, #b, (a), (b)))
#define EXPECT_NE(a, b) MG_GTEST_CHECK((a) != (b), ::testing::cmp_msg("!=", #a, #b, (a), (b)))
#define EXPECT_LT(a, b) MG_GTEST_CHECK((a) < (b), ::testing::cmp_msg("<", #a, #b, (a), (b)))
#define EXPECT_LE(a, b) MG_GTEST_CHECK((a) <= (b), ::testing::cmp_msg("<=", #a, #b, (a), (b)))
#define EXPECT_GT(a, b) MG_GTEST_CHECK((a) > (b), ::testing::cmp_msg(">", #a, #b, (a), (b)))
#define EXPECT_GE(a, b) MG_GTEST_CHECK((a) >= (b), ::testing::cmp_msg(">=", #a, #b, (a), (b)))
#define EXPECT_TRUE(c) MG_GTEST_CHECK((c), std::string("Expected true: ") + #c)
#define EXPECT_FALSE(c) MG_GTEST_CHECK(!(c), std::string("Expected false: ") + #c)
#define ASSERT_TRUE(c) MG_GTEST_CHECK_FATAL((c), std::string("Expected true: ") + #c)
#define EXPECT_DOUBLE_EQ(a, b) EXPECT_EQ(static_cast<double>(a), static_cast<double>(b))

#define EXPECT_THROW(stmt, extype)                                                                 \
  do {                                                                                             \
    bool mg_caught_ = false;                                                                       \
    try {                                                                                          \
      stmt;                                                                                        \
    } catch (const extype &) {                                                                     \
      mg_caught_ = true;                                                                           \
    } catch (...) {                                                                                \
    }                                                                                              \
    MG_GTEST_CHECK(mg_caught_, std::string("Expected ") + #stmt + " to throw " + #extype);         \
  } while (0)

#define EXPECT_NO_THROW(stmt)                                                                      \
  do {                                                                                             \
    bool mg_threw_ = false;                                                                        \
    try {                                                                                          \
      stmt;                                                                                        \
    } catch (...) {                                                                                \
      mg_threw_ = true;                                                                            \
    }                                                                                              \
    MG_GTEST_CHECK(!mg_threw_, std::string("Expected no throw: ") + #stmt);                        \
  } while (0)

#ifndef MG_GTEST_NO_MAIN
int main(int argc, char **argv) { return ::testing::run_all(argc, argv); }
#endif
