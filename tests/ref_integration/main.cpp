// Runner for the reference project's integration tests built against the stand-in
// gtest header in this folder.  Flags follow GoogleTest's names:
//   --also_run_disabled_tests   run tests whose name starts with DISABLED_
//   --gtest_filter=SUBSTRING    run only tests whose "Suite.Name" contains SUBSTRING
// Exit code: number of failed tests (0 = all passed or skipped).
#include <gtest/gtest.h>

#include <cstring>
#include <memory>
#include <string>

int main(int argc, char** argv) {
  bool runDisabled = false;
  std::string filter;
  for (int i = 1; i < argc; ++i) {
    if (!std::strcmp(argv[i], "--also_run_disabled_tests")) runDisabled = true;
    if (!std::strncmp(argv[i], "--gtest_filter=", 15)) filter = argv[i] + 15;
  }
  int ran = 0, failed = 0, skipped = 0, disabled = 0;
  for (auto& e : ::testing::internal::registry()) {
    std::string full = std::string(e.suite) + "." + e.name;
    if (!filter.empty() && full.find(filter) == std::string::npos) continue;
    if (!runDisabled && !std::strncmp(e.name, "DISABLED_", 9)) {
      ++disabled;
      continue;
    }
    std::printf("[ RUN      ] %s\n", full.c_str());
    std::fflush(stdout);
    int before = ::testing::internal::failures();
    std::unique_ptr<::testing::Test> t(e.make());
    t->SetUp();
    if (!t->skipped) t->TestBody();
    t->TearDown();
    ++ran;
    if (t->skipped) {
      ++skipped;
    } else if (::testing::internal::failures() != before) {
      ++failed;
      std::printf("[  FAILED  ] %s\n", full.c_str());
    } else {
      std::printf("[       OK ] %s\n", full.c_str());
    }
  }
  std::printf("[==========] %d ran, %d failed, %d skipped, %d disabled\n", ran, failed, skipped, disabled);
  return failed;
}
