// Minimal assertion harness for the C++ tests (GoogleTest is not available in this image).
#pragma once
#include <cmath>
#include <cstdio>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

namespace check
{
    struct Case { const char* name; std::function<void()> fn; };
    inline std::vector<Case>& cases() { static std::vector<Case> c; return c; }
    struct Register { Register(const char* n, std::function<void()> f) { cases().push_back({n, std::move(f)}); } };
    struct Failure : std::runtime_error { using std::runtime_error::runtime_error; };

    inline int run_all()
    {
        int failed = 0;
        for (auto& c : cases())
        {
            try { c.fn(); std::printf("[ OK ] %s\n", c.name); }
            catch (const std::exception& e) { ++failed; std::printf("[FAIL] %s: %s\n", c.name, e.what()); }
        }
        std::printf("%zu cases, %d failed\n", cases().size(), failed);
        return failed ? 1 : 0;
    }
}

#define TEST_CASE(name) \
    static void name(); \
    static check::Register reg_##name(#name, name); \
    static void name()

#define EXPECT_TRUE(cond) \
    do { if (!(cond)) throw check::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": " #cond); } while (0)

#define EXPECT_EQ(a, b) \
    do { if (!((a) == (b))) throw check::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": " #a " == " #b); } while (0)

#define EXPECT_NEAR(a, b, tol) \
    do { if (!(std::fabs(double(a) - double(b)) <= (tol))) throw check::Failure(std::string(__FILE__) + ":" + \
         std::to_string(__LINE__) + ": |" #a " - " #b "| = " + std::to_string(std::fabs(double(a) - double(b)))); } while (0)

#define EXPECT_THROWS(stmt, substr) \
    do { bool threw_ = false; \
         try { stmt; } catch (const std::runtime_error& e_) { threw_ = std::string(e_.what()).find(substr) != std::string::npos; \
               if (!threw_) throw check::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": wrong message: " + e_.what()); } \
         if (!threw_) throw check::Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": no exception from " #stmt); } while (0)
