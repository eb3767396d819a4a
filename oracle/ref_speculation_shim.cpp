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

// carat::select_placement over flat arrays: slot i's cached tokens are
// cached[offsets[i] .. offsets[i + 1]). Returns 0 placed, 1 no free slot, 2 reserve blocked.
#include "runtime/slot_policy.h"

extern "C" int ref_select_placement(const int *input_ids, int input_count, const int *cached,
                                    const int *offsets, const int *occupied,
                                    const unsigned long long *ages, const int *prefilling,
                                    int slot_count, int reserve, int *destination, int *source,
                                    unsigned long long *prefix_tokens) {
  std::vector<carat::SlotView> slots(static_cast<std::size_t>(slot_count));
  for (int index = 0; index < slot_count; ++index) {
    slots[static_cast<std::size_t>(index)] = carat::SlotView{
        .cached_tokens = std::span<const int>(
            cached + offsets[index], static_cast<std::size_t>(offsets[index + 1] - offsets[index])),
        .occupied = occupied[index] != 0,
        .age = ages[index],
        .prefilling = prefilling[index] != 0};
  }
  const auto decision = carat::select_placement(
      std::span<const int>(input_ids, static_cast<std::size_t>(input_count)), slots,
      static_cast<std::size_t>(reserve));
  if (const auto *placement = std::get_if<carat::Placement>(&decision)) {
    *destination = placement->destination;
    *source = placement->source.value_or(-1);
    *prefix_tokens = placement->prefix_tokens;
    return 0;
  }
  return std::holds_alternative<carat::NoFreeSlot>(decision) ? 1 : 2;
}
