// Minimal stand-in for the googletest API surface that the reference's own test file uses
// (reference tests/cpp/test_flash_attn.cu, tests/cpp/test.cpp): fixtures with SetUp/TearDown, TEST_F,
// ASSERT_EQ / EXPECT_TRUE with streamed messages, AssertionResult, GTEST_SKIP, InitGoogleTest, RUN_ALL_TESTS.
// googletest itself is an un-vendored submodule of the reference and is not installed here; with this header the
// reference's test sources compile UNCHANGED against include/flash_attn/flash_api.cuh (see build.sh beside it).
#pragma once

#include <cstdio>
#include <functional>
#include <sstream>
#include <string>
#include <vector>

namespace testing {

class AssertionResult {
 public:
  explicit AssertionResult(bool ok) : ok_(ok) {}
  AssertionResult(const AssertionResult& o) : ok_(o.ok_), msg_(o.msg_.str()) {}
  explicit operator bool() const { return ok_; }
  template <typename T>
  AssertionResult& operator<<(const T& v) {
    msg_ << v;
    return *this;
  }
  std::string message() const { return msg_.str(); }

 private:
  bool ok_;
  std::ostringstream msg_;
};
inline AssertionResult AssertionSuccess() { return AssertionResult(true); }
inline AssertionResult AssertionFailure() { return AssertionResult(false); }

class Test {
 public:
  virtual ~Test() {}
  virtual void SetUp() {}
  virtual void TearDown() {}
  virtual void TestBody() = 0;
  bool failed_ = false;
  bool skipped_ = false;
};

namespace internal {

struct Registry {
  struct Entry {
    std::string name;
    std::function<Test*()> make;
  };
  std::vector<Entry> tests;
  static Registry& get() {
    static Registry r;
    return r;
  }
};
struct Registrar {
  Registrar(const char* suite, const char* name, std::function<Test*()> make) {
    Registry::get().tests.push_back({std::string(suite) + "." + name, make});
  }
};

// Collects a streamed message and reports it when it goes out of scope.
class Reporter {
 public:
  Reporter(Test* t, const char* file, int line, const std::string& what, bool fatalOrFail, bool skip)
      : t_(t), skip_(skip) {
    msg_ << file << ":" << line << ": " << what;
    if (skip) {
      t_->skipped_ = true;
    } else if (fatalOrFail) {
      t_->failed_ = true;
    }
  }
  ~Reporter() { fprintf(stderr, "%s %s\n", skip_ ? "[ SKIPPED  ]" : "[ FAILURE  ]", msg_.str().c_str()); }
  template <typename T>
  Reporter& operator<<(const T& v) {
    msg_ << " " << v;
    return *this;
  }

 private:
  Test* t_;
  bool skip_;
  std::ostringstream msg_;
};
// `return Voidify() = Reporter(...) << ...;` lets a void function return after streaming
struct Voidify {
  void operator=(const Reporter&) {}
};

inline std::string describe(const AssertionResult& r) { return r.message(); }
inline std::string describe(bool) { return std::string(); }

}  // namespace internal

inline void InitGoogleTest(int*, char**) {}

}  // namespace testing

#define TEST_F(Fixture, Name)                                                                             \
  class Fixture##_##Name##_Test : public Fixture {                                                        \
   public:                                                                                                \
    void TestBody() override;                                                                             \
  };                                                                                                      \
  static ::testing::internal::Registrar registrar_##Fixture##_##Name(                                     \
      #Fixture, #Name, []() -> ::testing::Test* { return new Fixture##_##Name##_Test(); });               \
  void Fixture##_##Name##_Test::TestBody()

#define ASSERT_EQ(a, b)                                                                                   \
  if ((a) == (b))                                                                                         \
    ;                                                                                                     \
  else                                                                                                    \
    return ::testing::internal::Voidify() =                                                               \
               ::testing::internal::Reporter(this, __FILE__, __LINE__, "ASSERT_EQ(" #a ", " #b ") failed", true, false)

#define EXPECT_TRUE(expr)                                                                                 \
  if (auto gtest_res_ = (expr))                                                                           \
    ;                                                                                                     \
  else                                                                                                    \
    ::testing::internal::Reporter(this, __FILE__, __LINE__,                                               \
                                  std::string("EXPECT_TRUE(" #expr ") failed: ") +                        \
                                      ::testing::internal::describe(gtest_res_),                          \
                                  true, false)

#define GTEST_SKIP() \
  return ::testing::internal::Voidify() = ::testing::internal::Reporter(this, __FILE__, __LINE__, "skipped:", false, true)

inline int RUN_ALL_TESTS() {
  int passed = 0, failed = 0, skipped = 0;
  for (auto& e : ::testing::internal::Registry::get().tests) {
    ::testing::Test* t = e.make();
    t->SetUp();
    if (!t->skipped_ && !t->failed_) t->TestBody();
    t->TearDown();
    if (t->skipped_) {
      skipped++;
    } else if (t->failed_) {
      failed++;
      printf("[  FAILED  ] %s\n", e.name.c_str());
    } else {
      passed++;
      printf("[       OK ] %s\n", e.name.c_str());
    }
    delete t;
  }
  printf("[==========] %d tests: %d passed, %d failed, %d skipped\n", passed + failed + skipped, passed, failed, skipped);
  return failed == 0 ? 0 : 1;
}
