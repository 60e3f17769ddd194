// Activation-checkpoint planner: which decoder blocks to recompute so that the step fits a memory budget with the least
// extra compute.  Block i keeps `act[i]` bytes for its backward when stored, or `inp[i]` bytes (its input only) when
// checkpointed, in which case its forward (`cost[i]`) runs a second time and, while it is being recomputed, its full
// activations are live as well.  Minimise sum(cost of checkpointed blocks) subject to
//     sum_stored act + sum_ckpt inp + max_ckpt act <= budget.
// Solved exactly as a knapsack over `slots` memory quanta for every candidate "largest checkpointed block".
// The reference vendors a C dynamic program with the same purpose
// (colossalai auto_parallel/checkpoint/ckpt_solver_rotor.c), which none of its entry points use.
#include <cstdint>
#include <vector>

#define ATS_HOST_API extern "C" __attribute__((visibility("default")))

// flags[i] = 1 -> checkpoint block i.  Returns the extra cost, or -1 when even checkpointing everything does not fit.
ATS_HOST_API double ats_ckpt_plan(int n, const double* act, const double* inp, const double* cost, double budget, int slots, uint8_t* flags) {
  if (n <= 0 || slots < 1) return -1.0;
  double total_act = 0;
  for (int i = 0; i < n; ++i) total_act += act[i];
  for (int i = 0; i < n; ++i) flags[i] = 0;
  if (total_act <= budget) return 0.0;
  double best = -1.0;
  std::vector<uint8_t> best_flags(n, 0), take;
  const double INF = 1e300;
  // candidate peak = act[p]: only blocks with act <= act[p] may be checkpointed (ties broken by index), p itself is.
  for (int p = 0; p < n; ++p) {
    const double room = budget - act[p];  // what remains for the summed terms
    if (room < 0) continue;
    const double q = room / slots;
    if (q <= 0) continue;
    // saving (memory freed) of checkpointing i = act[i] - inp[i]; we need  total_act - sum_saving <= room
    const double need = total_act - room;
    // dp[s] = least cost to free at least s quanta; p is forced in.
    const int need_q = need <= 0 ? 0 : int(need / q) + 1;
    if (need_q > slots * 4) continue;
    std::vector<double> dp(need_q + 1, INF);
    std::vector<std::vector<uint8_t>> choice(n, std::vector<uint8_t>(need_q + 1, 0));
    auto quanta = [&](int i) { double s = act[i] - inp[i]; return s <= 0 ? 0 : int(s / q); };
    int forced = quanta(p);
    if (forced > need_q) forced = need_q;
    dp[forced] = cost[p];
    for (int s = 0; s < forced; ++s) dp[s] = cost[p];
    for (int i = 0; i < n; ++i) {
      if (i == p) continue;
      if (act[i] > act[p] || (act[i] == act[p] && i < p)) continue;
      const int w = quanta(i);
      if (w == 0) continue;
      for (int s = need_q; s >= 0; --s) {
        const int from = s - w < 0 ? 0 : s - w;
        if (dp[from] < INF && dp[from] + cost[i] < dp[s]) {
          dp[s] = dp[from] + cost[i];
          choice[i][s] = 1;
        }
      }
    }
    if (dp[need_q] >= INF) continue;
    if (best < 0 || dp[need_q] < best) {
      best = dp[need_q];
      take.assign(n, 0);
      take[p] = 1;
      int s = need_q;
      for (int i = n - 1; i >= 0; --i) {
        if (i == p || !choice[i][s]) continue;
        take[i] = 1;
        const int w = quanta(i);
        s = s - w < 0 ? 0 : s - w;
      }
      best_flags = take;
    }
  }
  if (best < 0) return -1.0;
  for (int i = 0; i < n; ++i) flags[i] = best_flags[i];
  return best;
}
