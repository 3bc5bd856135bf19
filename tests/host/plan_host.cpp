// Host build of the plan walker (mmaemu_b200/csrc/plan.cuh) for tests/test_plan_sequence_host.py.
#include "../../mmaemu_b200/csrc/plan.cuh"

// Writes the k-tile sequence of the plan (K, fast, S, scheme) into out (capacity entries) and returns its length, or
// the negated length when the capacity is too small.
extern "C" int plan_sequence_host(int K, int fast, int S, int scheme, uint32_t* out, int capacity) {
  const mmb::Plan plan = mmb::make_plan(K, fast, S, scheme);
  const int n = mmb::plan_sequence(plan, K, nullptr);
  if (n > capacity) return -n;
  return mmb::plan_sequence(plan, K, out);
}

// Chains of the plan's sequence and its cut into `slices` K slices; returns the number of chains (slice_start and
// chain_base hold slices + 1 entries; untouched when slices > chains or slices < 1).
extern "C" int plan_slices_host(int K, int fast, int S, int scheme, int slices, int* slice_start, int* chain_base) {
  const mmb::Plan plan = mmb::make_plan(K, fast, S, scheme);
  const int n = mmb::plan_sequence(plan, K, nullptr);
  uint32_t* seq = new uint32_t[n];
  mmb::plan_sequence(plan, K, seq);
  const int chains = mmb::plan_chains(seq, n, plan.group);
  if (slices >= 1 && slices <= chains) mmb::plan_slices(seq, n, plan.group, chains, slices, slice_start, chain_base);
  delete[] seq;
  return chains;
}

// The sequence written by `lanes` workers one after the other, as the threads of the device kernel write it together.
extern "C" int plan_sequence_lanes_host(int K, int fast, int S, int scheme, uint32_t* out, int capacity, int lanes) {
  const mmb::Plan plan = mmb::make_plan(K, fast, S, scheme);
  const int n = mmb::plan_sequence(plan, K, nullptr);
  if (n > capacity) return -n;
  for (int lane = 0; lane < lanes; ++lane)
    if (mmb::plan_sequence(plan, K, out, lane, lanes) != n) return 0;
  return n;
}
