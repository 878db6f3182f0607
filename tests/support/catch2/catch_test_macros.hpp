// A few-line stand-in for Catch2's TEST_CASE / REQUIRE macros, enough to compile
// llm-engine's own tests/test_block_allocator.cpp against this repository's
// KVCacheManager without the Catch2 dependency.  Test support only.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <string>
#include <utility>
#include <vector>

namespace mini_catch {
struct Registry {
  static std::vector<std::pair<std::string, std::function<void()>>>& cases() {
    static std::vector<std::pair<std::string, std::function<void()>>> c;
    return c;
  }
};
struct Registrar {
  Registrar(const char* name, std::function<void()> fn) { Registry::cases().emplace_back(name, std::move(fn)); }
};
inline int& failures() { static int f = 0; return f; }
}  // namespace mini_catch

#define MC_CAT2(a, b) a##b
#define MC_CAT(a, b) MC_CAT2(a, b)
#define TEST_CASE(...) \
  static void MC_CAT(mc_case_, __LINE__)(); \
  static mini_catch::Registrar MC_CAT(mc_reg_, __LINE__)(#__VA_ARGS__, MC_CAT(mc_case_, __LINE__)); \
  static void MC_CAT(mc_case_, __LINE__)()
#define REQUIRE(...) \
  do { if (!(__VA_ARGS__)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #__VA_ARGS__); mini_catch::failures()++; return; } } while (0)
#define REQUIRE_FALSE(...) \
  do { if ((__VA_ARGS__)) { std::printf("FAILED %s:%d: !(%s)\n", __FILE__, __LINE__, #__VA_ARGS__); mini_catch::failures()++; return; } } while (0)
#define CHECK(...) REQUIRE(__VA_ARGS__)

#ifdef MINI_CATCH_MAIN
int main() {
  for (auto& c : mini_catch::Registry::cases()) {
    const int before = mini_catch::failures();
    c.second();
    std::printf("%s %s\n", mini_catch::failures() == before ? "ok  " : "FAIL", c.first.c_str());
  }
  std::printf("cases=%zu failures=%d\n", mini_catch::Registry::cases().size(), mini_catch::failures());
  return mini_catch::failures() ? 1 : 0;
}
#endif
