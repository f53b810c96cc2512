// Minimal single-header test runner with the subset of the GoogleTest surface
// the reference's kernel tests use (TEST, EXPECT_LE/GE/EQ/NEAR/FLOAT_EQ with
// streamed messages).  GoogleTest itself is not available offline; this lets
// the reference's unmodified test sources be compiled and run against a
// replacement kernel library.  main() lives in runner_main.cpp.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

namespace rh_gtest_runner {

using TestFn = void (*)();

inline std::vector<std::pair<std::string, TestFn>>& registry() {
    static std::vector<std::pair<std::string, TestFn>> r;
    return r;
}
inline int& failure_count() {
    static int n = 0;
    return n;
}

struct Registrar {
    Registrar(const char* name, TestFn fn) { registry().emplace_back(name, fn); }
};

class Check {
public:
    Check(bool ok, const char* expr, const char* file, int line)
        : failed_(!ok), expr_(expr), file_(file), line_(line) {}
    Check(const Check&) = delete;
    ~Check() {
        if (failed_) {
            ++failure_count();
            std::fprintf(stderr, "%s:%d: Failure\n  expected: %s\n  %s\n", file_, line_, expr_,
                         msg_.str().c_str());
        }
    }
    template <class T>
    Check& operator<<(const T& v) {
        if (failed_) msg_ << v;
        return *this;
    }

private:
    bool failed_;
    const char* expr_;
    const char* file_;
    int line_;
    std::ostringstream msg_;
};

// `return Voidify() = Check(...) << msg;` — assignment binds looser than <<, so the message is streamed
// first and the whole expression has type void.
struct Voidify {
    void operator=(const Check&) const {}
};

// GoogleTest's EXPECT_FLOAT_EQ: equal within 4 units in the last place.
inline bool almost_equal_4ulp(float a, float b) {
    if (std::isnan(a) || std::isnan(b)) return false;
    auto biased = [](float f) {
        std::uint32_t u;
        std::memcpy(&u, &f, 4);
        return (u & 0x80000000u) ? (~u + 1) : (u | 0x80000000u);
    };
    std::uint32_t x = biased(a), y = biased(b);
    return (x > y ? x - y : y - x) <= 4;
}

inline int run_all() {
    for (auto& t : registry()) {
        int before = failure_count();
        std::printf("[ RUN      ] %s\n", t.first.c_str());
        t.second();
        std::printf("%s %s\n", failure_count() == before ? "[       OK ]" : "[  FAILED  ]",
                    t.first.c_str());
    }
    std::printf("%zu tests, %d failed expectations\n", registry().size(), failure_count());
    return failure_count() == 0 ? 0 : 1;
}

}  // namespace rh_gtest_runner

#define TEST(suite, name)                                                                  \
    static void suite##_##name##_body();                                                   \
    static ::rh_gtest_runner::Registrar suite##_##name##_registrar(#suite "." #name,       \
                                                                   &suite##_##name##_body); \
    static void suite##_##name##_body()

#define RH_CHECK_(cond, text) ::rh_gtest_runner::Check((cond), text, __FILE__, __LINE__)
#define EXPECT_LE(a, b) RH_CHECK_((a) <= (b), #a " <= " #b)
#define EXPECT_GE(a, b) RH_CHECK_((a) >= (b), #a " >= " #b)
#define EXPECT_LT(a, b) RH_CHECK_((a) < (b), #a " < " #b)
#define EXPECT_GT(a, b) RH_CHECK_((a) > (b), #a " > " #b)
#define EXPECT_EQ(a, b) RH_CHECK_((a) == (b), #a " == " #b)
#define EXPECT_NE(a, b) RH_CHECK_((a) != (b), #a " != " #b)
#define EXPECT_TRUE(a) RH_CHECK_(static_cast<bool>(a), #a)
#define EXPECT_FALSE(a) RH_CHECK_(!static_cast<bool>(a), "!(" #a ")")
#define EXPECT_FLOAT_EQ(a, b) RH_CHECK_(::rh_gtest_runner::almost_equal_4ulp((a), (b)), #a " ~= " #b)
// ASSERT_*: record the failure and leave the enclosing (void) function, like GoogleTest does.
#define ASSERT_EQ(a, b) \
    if ((a) == (b)) {} else return ::rh_gtest_runner::Voidify() = RH_CHECK_(false, #a " == " #b)
#define ASSERT_TRUE(a) \
    if (static_cast<bool>(a)) {} else return ::rh_gtest_runner::Voidify() = RH_CHECK_(false, #a)
#define EXPECT_NEAR(a, b, tol) RH_CHECK_(std::fabs((a) - (b)) <= (tol), "|" #a " - " #b "| <= " #tol)
