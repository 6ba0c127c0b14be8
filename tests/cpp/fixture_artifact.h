#pragma once
#include <cstdint>

constexpr std::uint64_t kFixtureWorkspaceBytes = 96;

struct FixtureObservation {
  int workspace_queries = 0;
  int runs = 0;
  bool fail_next_run = false;
  void* stream = nullptr;
  std::uint64_t flags = 0;
  void* workspace = nullptr;
  std::uint64_t workspace_size = 0;
  std::uint32_t num_values = 0;
};
