// A very small test runner (gtest is not available offline): TEST(name) registers a
// function; EXPECT/ASSERT macros record failures; main() runs the tests whose name
// contains the filter given on the command line.
#pragma once
#include <stdio.h>
#include <string.h>

#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

namespace mini {

struct Case {
    const char* name;
    std::function<void()> fn;
};
inline std::vector<Case>& cases() {
    static std::vector<Case> c;
    return c;
}
struct Registrar {
    Registrar(const char* name, std::function<void()> fn) { cases().push_back({name, std::move(fn)}); }
};
struct Failure : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct Skip : std::runtime_error {
    using std::runtime_error::runtime_error;
};
inline int& failures() {
    static int f = 0;
    return f;
}

inline int run_all(const char* filter) {
    int ran = 0, failed = 0, skipped = 0;
    for (auto& c : cases()) {
        if (filter != nullptr && strstr(c.name, filter) == nullptr)
            continue;
        const int before = failures();
        bool skip = false;
        try {
            c.fn();
        } catch (const Skip& s) {
            skip = true;
            printf("[ SKIPPED ] %s: %s\n", c.name, s.what());
        } catch (const std::exception& e) {
            ++failures();
            printf("  exception: %s\n", e.what());
        }
        ++ran;
        if (skip) {
            ++skipped;
        } else if (failures() != before) {
            ++failed;
            printf("[ FAILED  ] %s\n", c.name);
        } else {
            printf("[   OK    ] %s\n", c.name);
        }
        fflush(stdout);
    }
    printf("%d tests, %d failed, %d skipped\n", ran, failed, skipped);
    return failed == 0 ? 0 : 1;
}

}  // namespace mini

#define TEST(name)                                                  \
    static void test_##name();                                      \
    static mini::Registrar registrar_##name(#name, test_##name);    \
    static void test_##name()

#define EXPECT_TRUE(cond)                                                              \
    do {                                                                               \
        if (!(cond)) {                                                                 \
            ++mini::failures();                                                        \
            printf("  %s:%d: expected %s\n", __FILE__, __LINE__, #cond);               \
        }                                                                              \
    } while (0)

#define EXPECT_EQ(a, b)                                                                \
    do {                                                                               \
        if (!((a) == (b))) {                                                           \
            ++mini::failures();                                                        \
            printf("  %s:%d: %s != %s\n", __FILE__, __LINE__, #a, #b);                 \
        }                                                                              \
    } while (0)

#define ASSERT_TRUE(cond)                                                              \
    do {                                                                               \
        if (!(cond))                                                                   \
            throw mini::Failure(std::string(#cond) + " at " + __FILE__ + ":" + std::to_string(__LINE__)); \
    } while (0)

#define SKIP(msg) throw mini::Skip(msg)
