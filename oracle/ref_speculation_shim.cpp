// C wrapper around the reference's own speculation logic (src/runtime/speculation.{h,cpp}), so
// Python tests and bench.py's reference arm can call the unmodified reference code.
// TEST INFRASTRUCTURE. Built by oracle/Makefile into oracle/_ref/ from the sources where they lie
// in the reference tree; no reference source is copied into this repository.
#include "runtime/speculation.h"

#include <span>
#include <unordered_set>
#include <vector>

extern "C" int ref_acceptance_cap(int depth, int remaining, const int *proposals,
                                  int proposal_count, const int *stop_ids, int stop_count) {
  const std::unordered_set<int> stops(stop_ids, stop_ids + stop_count);
  return carat::acceptance_cap(
      depth, remaining, std::span<const int>(proposals, static_cast<std::size_t>(proposal_count)),
      stops);
}

extern "C" int ref_commit_speculation(int forced_token, const int *accepted_drafts,
                                      int accepted_count, int next_token, const int *stop_ids,
                                      int stop_count, int *resident, int *resident_count,
                                      int *emitted, int *emitted_count, int *next_out) {
  const std::unordered_set<int> stops(stop_ids, stop_ids + stop_count);
  const auto commit = carat::commit_speculation(
      forced_token,
      std::span<const int>(accepted_drafts, static_cast<std::size_t>(accepted_count)), next_token,
      stops);
  for (std::size_t index = 0; index < commit.resident_tokens.size(); ++index)
    resident[index] = commit.resident_tokens[index];
  for (std::size_t index = 0; index < commit.emitted_tokens.size(); ++index)
    emitted[index] = commit.emitted_tokens[index];
  *resident_count = static_cast<int>(commit.resident_tokens.size());
  *emitted_count = static_cast<int>(commit.emitted_tokens.size());
  *next_out = commit.next_token;
  return commit.stopped ? 1 : 0;
}
