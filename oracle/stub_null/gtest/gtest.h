// Stand-in for <gtest/gtest.h> used only to reach the host-side reference
// helpers that live in the anonymous namespaces of the reference's kernel test
// sources.  TEST bodies become function templates that are never instantiated,
// so nothing that launches a GPU kernel is emitted; EXPECT_* swallow their
// operands.
#pragma once

namespace rh_gtest_null {
struct Sink {
    template <class T>
    const Sink& operator<<(const T&) const { return *this; }
};
}  // namespace rh_gtest_null

#define TEST(suite, name) \
    template <int> [[maybe_unused]] static void suite##_##name##_never_instantiated()

#define RH_NULL_EXPECT(...) ::rh_gtest_null::Sink()
#define EXPECT_LE(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_GE(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_LT(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_GT(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_EQ(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_NE(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_TRUE(a) RH_NULL_EXPECT(a)
#define EXPECT_FALSE(a) RH_NULL_EXPECT(a)
#define EXPECT_FLOAT_EQ(a, b) RH_NULL_EXPECT(a, b)
#define EXPECT_NEAR(a, b, tol) RH_NULL_EXPECT(a, b, tol)
#define ASSERT_EQ(a, b) RH_NULL_EXPECT(a, b)
#define ASSERT_TRUE(a) RH_NULL_EXPECT(a)
