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
