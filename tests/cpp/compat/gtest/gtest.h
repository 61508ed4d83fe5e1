// A minimal stand-in for the typed-test subset of a unit-test framework's <gtest/gtest.h>, just
// large enough to compile and run the reference's typed GEMM tests unmodified
// (test/gemm/test_float_accum.cpp, test/gemm/test_same_prec.cpp of adelj88/rocm_wmma_gemm):
// fixtures derived from ::testing::Test, ::testing::Types<...>, TYPED_TEST_SUITE, TYPED_TEST,
// ASSERT_EQ / ASSERT_NEAR / ASSERT_GT with a streamed message, InitGoogleTest, RUN_ALL_TESTS.
// Written for this repository; the real framework is not available offline.  Test infrastructure.
#ifndef B200_COMPAT_GTEST_H
#define B200_COMPAT_GTEST_H

#include <cmath>
#include <cstdio>
#include <functional>
#include <sstream>
#include <string>
#include <vector>

namespace testing {

class Test {
public:
    virtual ~Test() = default;
    void Run()
    {
        SetUp();
        TestBody();
        TearDown();
    }

protected:
    virtual void SetUp() {}
    virtual void TearDown() {}
    virtual void TestBody() = 0;
};

template <class... Ts>
struct Types {};

namespace internal {

struct Case {
    std::string            name;
    std::function<Test*()> make;
};
inline std::vector<Case>& registry()
{
    static std::vector<Case> r;
    return r;
}
inline bool& current_failed()
{
    static bool f = false;
    return f;
}

struct Message {
    std::ostringstream ss;
    template <class T>
    Message& operator<<(const T& v)
    {
        ss << v;
        return *this;
    }
};

// `return AssertHelper(...) = Message() << ...;` records the failure and leaves the (void) test body.
struct AssertHelper {
    const char* file;
    int         line;
    std::string what;
    void operator=(const Message& m) const
    {
        current_failed() = true;
        std::printf("%s:%d: failure: %s %s\n", file, line, what.c_str(), m.ss.str().c_str());
    }
};

template <template <class> class TestT, class List>
struct RegisterTyped;
template <template <class> class TestT, class... Ts>
struct RegisterTyped<TestT, Types<Ts...>> {
    explicit RegisterTyped(const char* name)
    {
        int index = 0;
        (registry().push_back(Case{std::string(name) + "/" + std::to_string(index++), []() -> Test* { return new TestT<Ts>; }}), ...);
    }
};

} // namespace internal

inline void InitGoogleTest(int*, char**) {}

inline int RunAllTests()
{
    int ran = 0, failed = 0;
    for (auto& c : internal::registry()) {
        internal::current_failed() = false;
        Test* t                    = c.make();
        t->Run();
        delete t;
        ++ran;
        if (internal::current_failed()) {
            ++failed;
            std::printf("[  FAILED  ] %s\n", c.name.c_str());
        }
    }
    std::printf("%d tests ran, %d failed\n", ran, failed);
    return failed ? 1 : 0;
}

} // namespace testing

#define RUN_ALL_TESTS() ::testing::RunAllTests()

#define TYPED_TEST_SUITE(Suite, TypeList) typedef TypeList gtest_types_##Suite

#define TYPED_TEST(Suite, Name)                                                                              \
    template <class gtest_TypeParam>                                                                         \
    class Suite##_##Name##_Test : public Suite<gtest_TypeParam> {                                            \
        typedef Suite<gtest_TypeParam> TestFixture;                                                          \
        typedef gtest_TypeParam        TypeParam;                                                            \
        void                           TestBody() override;                                                  \
    };                                                                                                       \
    static ::testing::internal::RegisterTyped<Suite##_##Name##_Test, gtest_types_##Suite> gtest_reg_##Suite##_##Name( \
        #Suite "." #Name);                                                                                   \
    template <class gtest_TypeParam>                                                                         \
    void Suite##_##Name##_Test<gtest_TypeParam>::TestBody()

#define B200_GTEST_FAIL_(text) \
    return ::testing::internal::AssertHelper{__FILE__, __LINE__, text} = ::testing::internal::Message()

#define ASSERT_EQ(a, b) \
    if ((a) == (b)) {   \
    } else              \
        B200_GTEST_FAIL_("ASSERT_EQ(" #a ", " #b ")")
#define ASSERT_GT(a, b) \
    if ((a) > (b)) {    \
    } else              \
        B200_GTEST_FAIL_("ASSERT_GT(" #a ", " #b ")")
#define ASSERT_NEAR(a, b, tol)                                                      \
    if (std::fabs(static_cast<double>(a) - static_cast<double>(b)) <= (tol)) {     \
    } else                                                                          \
        B200_GTEST_FAIL_("ASSERT_NEAR(" #a ", " #b ", " #tol ")")
#define ASSERT_TRUE(c) \
    if (c) {           \
    } else             \
        B200_GTEST_FAIL_("ASSERT_TRUE(" #c ")")

#endif // B200_COMPAT_GTEST_H
