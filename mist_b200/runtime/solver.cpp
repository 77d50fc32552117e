// Host-side native runtime of the tuner: Pareto sampling of (stable, delta) cost pairs,
// the exact inter-stage solver, and an event-driven 1F1B pipeline simulator.
//
// The reference solves the inter-stage problem as a MILP through PuLP + a CBC subprocess
// (mist/analyzer/inter_tuning_mip.py:308-425) and samples Pareto points with numba
// (mist/utils/pareto.py:8-148).  The problem is small and has a clean structure, so it is
// solved exactly here by dynamic programming over (stage, layers used) with a Pareto
// front of (sum of stage times, worst exposed delta) per state, once per candidate value
// of the bottleneck stage time.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <queue>
#include <vector>

#define RT_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------- Pareto
// For `samples` weights alpha in (0,1), picks argmin alpha/(1-alpha) * stable + delta over
// feasible candidates.  out_idx gets `samples` indices (-1 when nothing is feasible).
RT_API int rt_pareto_sample(const double* stable, const double* delta, const uint8_t* feasible, int64_t n,
                            int samples, int64_t* out_idx) {
  for (int s = 0; s < samples; ++s) {
    const double alpha = static_cast<double>(s + 1) / static_cast<double>(samples + 1);
    const double w = alpha / (1.0 - alpha);
    double best = std::numeric_limits<double>::infinity();
    int64_t arg = -1;
    for (int64_t i = 0; i < n; ++i) {
      if (feasible && !feasible[i]) continue;
      const double v = w * stable[i] + delta[i];
      if (v < best) {
        best = v;
        arg = i;
      }
    }
    out_idx[s] = arg;
  }
  return 0;
}

// --------------------------------------------------------------------- inter-stage DP
namespace {

struct Option {
  int kind;      // 0 first, 1 any middle stage, 2 last, 3 only stage, 10 + s the middle stage at index s
  int layers;
  double T, D;
  int id;        // caller's identifier
};

struct Label {
  double sumT, worst;
  int prev_layers;   // layers used before this stage
  int prev_label;    // index into the previous state's front
  int option;        // index into the option array
};

inline bool dominates(const Label& a, const Label& b) { return a.sumT <= b.sumT && a.worst <= b.worst; }

void insert_label(std::vector<Label>& front, const Label& l, size_t cap) {
  for (const Label& f : front)
    if (dominates(f, l)) return;
  front.erase(std::remove_if(front.begin(), front.end(), [&](const Label& f) { return dominates(l, f); }),
              front.end());
  front.push_back(l);
  if (front.size() > cap) {
    // keep the labels with the smallest sumT + max(worst, 0): a bounded beam, exact for small fronts
    std::sort(front.begin(), front.end(), [](const Label& a, const Label& b) {
      return a.sumT + std::max(a.worst, 0.0) < b.sumT + std::max(b.worst, 0.0);
    });
    front.resize(cap);
  }
}

}  // namespace

// Chooses one option per stage (stage 0 must be kind first/only, the last stage kind last/only,
// the others middle) so that the layer counts add up to `total_layers`, minimising
//     (G - 1) * max_s T_s + sum_s T_s + max(0, max_s (D_s - sum_{j<s} T_j)).
// Returns the optimal cost (infinity when infeasible) and writes the chosen option ids.
RT_API double rt_inter_stage_solve(int num_stages, int total_layers, int grad_accum, int64_t num_options,
                                   const int32_t* opt_kind, const int32_t* opt_layers, const double* opt_T,
                                   const double* opt_D, const int32_t* opt_id, int32_t* chosen_ids) {
  std::vector<Option> opts(num_options);
  std::vector<double> tvals;
  for (int64_t i = 0; i < num_options; ++i) {
    opts[i] = {opt_kind[i], opt_layers[i], opt_T[i], opt_D[i], opt_id[i]};
    if (std::isfinite(opt_T[i])) tvals.push_back(opt_T[i]);
  }
  std::sort(tvals.begin(), tvals.end());
  tvals.erase(std::unique(tvals.begin(), tvals.end()), tvals.end());
  const double inf = std::numeric_limits<double>::infinity();
  double best_cost = inf;
  std::vector<int> best_choice;

  auto kind_of_stage = [&](int s) {
    if (num_stages == 1) return 3;
    if (s == 0) return 0;
    if (s == num_stages - 1) return 2;
    return 1;
  };
  // options grouped per stage kind; a middle stage takes the options priced for exactly its index (kind 10 + s:
  // its own 1F1B warm-up depth) when the caller supplied some, else the ones priced for any middle stage
  constexpr int kExact = 10;
  std::vector<std::vector<int>> by_kind(kExact + num_stages);
  for (int i = 0; i < static_cast<int>(opts.size()); ++i)
    if (opts[i].kind >= 0 && opts[i].kind < static_cast<int>(by_kind.size()) && std::isfinite(opts[i].T))
      by_kind[opts[i].kind].push_back(i);
  auto candidates_of_stage = [&](int s) -> const std::vector<int>& {
    const int k = kind_of_stage(s);
    if (k == 1 && !by_kind[kExact + s].empty()) return by_kind[kExact + s];
    return by_kind[k];
  };

  const size_t kFrontCap = 64;
  for (double tmax : tvals) {
    if ((grad_accum - 1) * tmax >= best_cost) break;   // larger bottlenecks cannot win any more
    // fronts[s][layers_used]
    std::vector<std::vector<std::vector<Label>>> fronts(
        num_stages + 1, std::vector<std::vector<Label>>(total_layers + 1));
    fronts[0][0].push_back({0.0, -inf, -1, -1, -1});
    bool uses_tmax = false;
    for (int s = 0; s < num_stages; ++s) {
      const auto& cand = candidates_of_stage(s);
      for (int used = 0; used <= total_layers; ++used) {
        const auto& cur = fronts[s][used];
        if (cur.empty()) continue;
        for (int oi : cand) {
          const Option& o = opts[oi];
          if (o.T > tmax) continue;
          const int nu = used + o.layers;
          if (nu > total_layers) continue;
          // remaining stages need at least one layer each
          if (total_layers - nu < (num_stages - 1 - s)) continue;
          for (int li = 0; li < static_cast<int>(cur.size()); ++li) {
            Label nl{cur[li].sumT + o.T, std::max(cur[li].worst, o.D - cur[li].sumT), used, li, oi};
            insert_label(fronts[s + 1][nu], nl, kFrontCap);
          }
        }
      }
    }
    const auto& fin = fronts[num_stages][total_layers];
    for (int li = 0; li < static_cast<int>(fin.size()); ++li) {
      // reconstruct to learn the true bottleneck of this assignment
      std::vector<int> choice(num_stages);
      int layers = total_layers, lab = li;
      double real_max = 0.0;
      for (int s = num_stages; s >= 1; --s) {
        const Label& l = fronts[s][layers][lab];
        choice[s - 1] = l.option;
        real_max = std::max(real_max, opts[l.option].T);
        layers = l.prev_layers;
        lab = l.prev_label;
      }
      const Label& f = fin[li];
      const double cost = (grad_accum - 1) * real_max + f.sumT + std::max(f.worst, 0.0);
      if (cost < best_cost) {
        best_cost = cost;
        best_choice = choice;
      }
      (void)uses_tmax;
    }
  }
  if (best_choice.empty()) return inf;
  for (int s = 0; s < num_stages; ++s) chosen_ids[s] = opts[best_choice[s]].id;
  return best_cost;
}

// ------------------------------------------------------------------- 1F1B simulation
// Event-driven simulation of a non-interleaved 1F1B schedule with `S` stages and `G` micro
// batches: per-stage forward / backward times, a p2p transfer time between neighbours and a
// once-per-iteration tail per stage.  Returns the iteration time; `stage_busy` (may be null)
// receives each stage's total busy time.
RT_API double rt_simulate_1f1b(int S, int G, const double* fwd, const double* bwd, const double* delta,
                               double p2p, double* stage_busy) {
  // op order per stage: warm-up forwards, then alternating (F, B), then cool-down backwards
  std::vector<std::vector<std::pair<char, int>>> order(S);
  for (int s = 0; s < S; ++s) {
    const int warm = std::min(S - 1 - s, G);
    int f = 0, b = 0;
    for (int i = 0; i < warm; ++i) order[s].push_back({'F', f++});
    while (f < G) {
      order[s].push_back({'F', f++});
      order[s].push_back({'B', b++});
    }
    while (b < G) order[s].push_back({'B', b++});
  }
  const double inf = std::numeric_limits<double>::infinity();
  std::vector<std::vector<double>> f_done(S, std::vector<double>(G, inf)), b_done(S, std::vector<double>(G, inf));
  std::vector<size_t> pos(S, 0);
  std::vector<double> free_at(S, 0.0), busy(S, 0.0);
  bool progress = true;
  while (progress) {
    progress = false;
    for (int s = 0; s < S; ++s) {
      while (pos[s] < order[s].size()) {
        auto [kind, mb] = order[s][pos[s]];
        double ready;
        if (kind == 'F') ready = (s == 0) ? 0.0 : f_done[s - 1][mb] + p2p;
        else ready = (s == S - 1) ? f_done[s][mb] : b_done[s + 1][mb] + p2p;
        if (!std::isfinite(ready)) break;
        const double start = std::max(ready, free_at[s]);
        const double dur = (kind == 'F') ? fwd[s] : bwd[s];
        free_at[s] = start + dur;
        busy[s] += dur;
        if (kind == 'F') f_done[s][mb] = free_at[s];
        else b_done[s][mb] = free_at[s];
        ++pos[s];
        progress = true;
      }
    }
  }
  double end = 0.0;
  for (int s = 0; s < S; ++s) {
    if (pos[s] != order[s].size()) return -1.0;   // should not happen: the schedule is deadlock free
    end = std::max(end, free_at[s] + (delta ? delta[s] : 0.0));
    if (stage_busy) stage_busy[s] = busy[s];
  }
  return end;
}

// ---------------------------------------------------------------- copy-engine planner
// Splits host<->device transfers into chunks and orders them by deadline so that a copy
// needed soon is never stuck behind a large one (used by the offload engine).  Inputs:
// per transfer its size, earliest start and deadline (seconds); output: chunk list
// (transfer index, offset, bytes) in issue order.  Returns the number of chunks written.
RT_API int64_t rt_plan_copy_chunks(int64_t n, const int64_t* bytes, const double* ready, const double* deadline,
                                   int64_t chunk_bytes, int64_t max_chunks, int64_t* out_transfer,
                                   int64_t* out_offset, int64_t* out_bytes) {
  struct Item {
    double deadline, ready;
    int64_t idx;
  };
  std::vector<Item> items;
  for (int64_t i = 0; i < n; ++i) items.push_back({deadline[i], ready[i], i});
  std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) {
    if (a.deadline != b.deadline) return a.deadline < b.deadline;
    return a.ready < b.ready;
  });
  std::vector<int64_t> done(n, 0);
  int64_t count = 0;
  bool left = true;
  // round-robin over transfers in deadline order, one chunk at a time from the two most urgent
  while (left && count < max_chunks) {
    left = false;
    int served = 0;
    for (const Item& it : items) {
      if (done[it.idx] >= bytes[it.idx]) continue;
      left = true;
      const int64_t sz = std::min(chunk_bytes, bytes[it.idx] - done[it.idx]);
      out_transfer[count] = it.idx;
      out_offset[count] = done[it.idx];
      out_bytes[count] = sz;
      done[it.idx] += sz;
      ++count;
      if (++served == 2 || count >= max_chunks) break;
    }
  }
  return count;
}
