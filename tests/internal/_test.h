// Minimal test runner for the torch-free C++ components.
#pragma once
#include <cstdio>
#include <exception>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

struct TestCase { const char* name; std::function<void()> fn; };
inline std::vector<TestCase>& test_registry() { static std::vector<TestCase> r; return r; }
struct TestRegistrar { TestRegistrar(const char* n, std::function<void()> f) { test_registry().push_back({n, std::move(f)}); } };
#define TEST_CASE(name) static void name(); static TestRegistrar reg_##name(#name, name); static void name()
#define CHECK(cond) do { if (!(cond)) { std::fprintf(stderr, "  CHECK failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__); throw std::runtime_error("check failed"); } } while (0)
inline int run_all_tests() {
  int failed = 0;
  for (auto& t : test_registry()) {
    try { t.fn(); std::printf("[ ok ] %s\n", t.name); }
    catch (const std::exception& e) { std::printf("[FAIL] %s: %s\n", t.name, e.what()); ++failed; }
  }
  std::printf("%zu tests, %d failed\n", test_registry().size(), failed);
  return failed ? 1 : 0;
}
