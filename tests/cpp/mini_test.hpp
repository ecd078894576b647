// A tiny test harness (gtest is not available offline): TEST(name) registers a
// function, CHECK / CHECK_EQ / CHECK_THROWS_STATUS record failures, main() runs
// every test (or those whose name contains argv[1]) and exits nonzero on failure.
#ifndef FTRAIN_TESTS_MINI_TEST_HPP_
#define FTRAIN_TESTS_MINI_TEST_HPP_

#include <cstdio>
#include <cstring>
#include <functional>
#include <sstream>
#include <string>
#include <vector>

#include "core/error.hpp"

namespace mini {

struct Case {
    const char* name;
    std::function<void()> body;
};

inline std::vector<Case>& registry() {
    static std::vector<Case> cases;
    return cases;
}

inline int& failures() {
    static int count = 0;
    return count;
}

struct Registrar {
    Registrar(const char* name, std::function<void()> body) { registry().push_back(Case{name, std::move(body)}); }
};

inline void fail(const char* file, int line, const std::string& what) {
    ++failures();
    std::printf("    FAILED %s:%d: %s\n", file, line, what.c_str());
}

template<typename A, typename B>
void checkEq(const A& a, const B& b, const char* a_text, const char* b_text, const char* file, int line) {
    if (!(a == b)) {
        std::ostringstream out;
        out << a_text << " == " << b_text << " (" << a << " vs " << b << ")";
        fail(file, line, out.str());
    }
}

inline int runAll(int argc, char** argv) {
    const char* filter = argc > 1 ? argv[1] : "";
    int ran            = 0;
    for (const Case& test : registry()) {
        if (std::strstr(test.name, filter) == nullptr) { continue; }
        const int before = failures();
        try {
            test.body();
        } catch (const std::exception& error) {
            fail(test.name, 0, std::string("unexpected exception: ") + error.what());
        } catch (...) { fail(test.name, 0, "unexpected non-standard exception"); }
        std::printf("[%s] %s\n", failures() == before ? " ok " : "FAIL", test.name);
        ++ran;
    }
    std::printf("%d tests, %d failed checks\n", ran, failures());
    return failures() == 0 && ran > 0 ? 0 : 1;
}

}  // namespace mini

#define TEST(name)                                                   \
    static void test_##name();                                       \
    static ::mini::Registrar registrar_##name(#name, test_##name);   \
    static void test_##name()

#define CHECK(condition)                                                          \
    do {                                                                          \
        if (!(condition)) { ::mini::fail(__FILE__, __LINE__, #condition); }       \
    } while (0)

#define CHECK_EQ(a, b) ::mini::checkEq((a), (b), #a, #b, __FILE__, __LINE__)

// The statement must throw ftrain::Exception carrying `status`.
#define CHECK_THROWS_STATUS(statement, status)                                                          \
    do {                                                                                                \
        bool threw_ = false;                                                                            \
        try {                                                                                           \
            statement;                                                                                  \
        } catch (const ::ftrain::Exception& error_) {                                                   \
            threw_ = true;                                                                              \
            CHECK_EQ(static_cast<int>(error_.getResult().getStatus()), static_cast<int>(status));       \
        }                                                                                               \
        if (!threw_) { ::mini::fail(__FILE__, __LINE__, #statement " did not throw"); }                 \
    } while (0)

#endif
