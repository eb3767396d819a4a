// Where a new request goes: the slot inside one replica (the reference's placement rule) and the
// replica inside the box (which the reference, a single-GPU server, does not have).
//
// Inside a replica the rule is carat::select_placement (src/runtime/slot_policy.cpp:22-84):
// reuse the longest cached prefix, in place when its slot is idle, else by cloning into an
// empty slot, else by evicting the oldest idle cache unless the idle-cache reserve forbids it.
// Across replicas a request goes where it reuses the most cached tokens; ties go to the replica
// with the least work (occupied slots plus queued requests), then to the lowest index. A request
// never moves once placed, and slots never migrate between GPUs: replicas share nothing.
#include "../../include/carat_b200.h"
#include "context.cuh"

#include <cstddef>
#include <cstdint>

using namespace carat_b200;

namespace {

bool reuses_cache(const int *input_ids, int input_count, const carat_b200_slot_view &slot) {
  if (slot.cached_count <= 0 || slot.cached_count > input_count)
    return false;
  if (slot.cached_count == input_count && slot.prefilling != 0)
    return false;   // a prefilling slot has no prediction after its cached prefix yet
  for (int index = 0; index < slot.cached_count; ++index) {
    if (slot.cached_tokens[index] != input_ids[index])
      return false;
  }
  return true;
}

// The single-replica decision, written out as one pass over the slots for each of the three
// questions the rule asks (best source, an empty slot, the eviction victim).
carat_b200_placement place_in_replica(const int *input_ids, int input_count,
                                      const carat_b200_slot_view *slots, int slot_count,
                                      int idle_cache_reserve_slots) {
  carat_b200_placement result{};
  result.decision = CARAT_B200_NO_FREE_SLOT;
  result.source = -1;
  int source = -1;
  int prefix = 0;
  for (int index = 0; index < slot_count; ++index) {
    if (!reuses_cache(input_ids, input_count, slots[index]))
      continue;
    const bool longer = slots[index].cached_count > prefix;
    const bool idle_beats_busy = slots[index].cached_count == prefix && source >= 0 &&
                                 slots[source].occupied != 0 && slots[index].occupied == 0;
    if (longer || idle_beats_busy) {
      source = index;
      prefix = slots[index].cached_count;
    }
  }
  result.source = source;
  result.prefix_tokens = static_cast<uint64_t>(prefix);
  if (source >= 0 && slots[source].occupied == 0) {
    result.decision = CARAT_B200_PLACED;
    result.destination = source;
    return result;
  }
  for (int index = 0; index < slot_count; ++index) {
    if (slots[index].occupied == 0 && slots[index].cached_count <= 0) {
      result.decision = CARAT_B200_PLACED;
      result.destination = index;
      return result;
    }
  }
  int victim = -1;
  int active = 0;
  int idle_cached = 0;
  for (int index = 0; index < slot_count; ++index) {
    if (slots[index].occupied != 0) {
      ++active;
      continue;
    }
    ++idle_cached;
    if (victim < 0 || slots[index].age < slots[victim].age)
      victim = index;
  }
  if (victim < 0)
    return result;
  if (active > 0 && idle_cached <= idle_cache_reserve_slots &&
      prefix < slots[victim].cached_count) {
    result.decision = CARAT_B200_RESERVE_BLOCKED;
    return result;
  }
  result.decision = CARAT_B200_PLACED;
  result.destination = victim;
  return result;
}

} // namespace

extern "C" int carat_b200_select_placement(const int *input_ids, int input_count,
                                           const carat_b200_slot_view *slots, int slot_count,
                                           int idle_cache_reserve_slots,
                                           carat_b200_placement *placement) {
  if (input_ids == nullptr || input_count <= 0 || slots == nullptr || slot_count <= 0 ||
      idle_cache_reserve_slots < 0 || placement == nullptr) {
    set_last_error("invalid placement request");
    return -1;
  }
  *placement = place_in_replica(input_ids, input_count, slots, slot_count,
                                idle_cache_reserve_slots);
  placement->replica = 0;
  return 0;
}

extern "C" int carat_b200_route_request(const int *input_ids, int input_count,
                                        const carat_b200_replica_view *replicas, int replica_count,
                                        int idle_cache_reserve_slots,
                                        carat_b200_placement *placement) {
  if (input_ids == nullptr || input_count <= 0 || replicas == nullptr || replica_count <= 0 ||
      idle_cache_reserve_slots < 0 || placement == nullptr) {
    set_last_error("invalid placement request");
    return -1;
  }
  carat_b200_placement best{};
  best.decision = CARAT_B200_NO_FREE_SLOT;
  best.replica = -1;
  best.source = -1;
  long long best_load = 0;
  bool blocked = false;
  for (int replica = 0; replica < replica_count; ++replica) {
    const carat_b200_replica_view &view = replicas[replica];
    if (view.alive == 0 || view.slots == nullptr || view.slot_count <= 0)
      continue;
    carat_b200_placement candidate = place_in_replica(input_ids, input_count, view.slots,
                                                      view.slot_count, idle_cache_reserve_slots);
    if (candidate.decision == CARAT_B200_RESERVE_BLOCKED)
      blocked = true;
    if (candidate.decision != CARAT_B200_PLACED)
      continue;
    long long load = view.queued_requests;
    for (int index = 0; index < view.slot_count; ++index)
      load += view.slots[index].occupied != 0 ? 1 : 0;
    candidate.replica = replica;
    const bool better = best.replica < 0 || candidate.prefix_tokens > best.prefix_tokens ||
                        (candidate.prefix_tokens == best.prefix_tokens && load < best_load);
    if (better) {
      best = candidate;
      best_load = load;
    }
  }
  if (best.replica < 0 && blocked)
    best.decision = CARAT_B200_RESERVE_BLOCKED;
  *placement = best;
  return 0;
}
