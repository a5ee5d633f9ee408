// Pipeline-parallel schedules (GPipe, 1F1B, interleaved 1F1B, ZB-H1): the action list of a rank, the closed-form
// bubble fractions, the balanced contiguous partition of layer costs and an event-driven simulation of a schedule.
// The model is cut into pp * v chunks; chunk g lives on rank g % pp.  For every chunk the backward actions visit the
// micro-batches in increasing order, so gradient accumulation order is the same for every schedule.
// Parity: include/nexus/dist/pipeline.hpp and src/dist/pipeline.cpp of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <deque>
#include <limits>
#include <map>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace py = pybind11;

namespace {

enum Kind : int { kF = 0, kB = 1 };
struct Action { int kind; int mb; int chunk; };
enum Sched : int { kGpipe, k1f1b, kInterleaved, kZbH1 };

Sched parse(const std::string& name) {
  if (name == "gpipe") return kGpipe;
  if (name == "1f1b") return k1f1b;
  if (name == "interleaved_1f1b") return kInterleaved;
  if (name == "zb_h1") return kZbH1;
  throw std::invalid_argument("unknown pipeline schedule '" + name + "'");
}

std::vector<Action> make(const std::string& name, int pp, int rank, int m, int v) {
  const Sched s = parse(name);
  if (pp < 1 || rank < 0 || rank >= pp || m < 1 || v < 1)
    throw std::invalid_argument("make_schedule: pp >= 1, 0 <= rank < pp, microbatches >= 1, virtual_stages >= 1");
  std::vector<Action> acts;
  if (s == kGpipe) {
    for (int c = 0; c < v; ++c)
      for (int i = 0; i < m; ++i) acts.push_back({kF, i, c * pp + rank});
    for (int c = v - 1; c >= 0; --c)
      for (int i = 0; i < m; ++i) acts.push_back({kB, i, c * pp + rank});
    return acts;
  }
  if (s == k1f1b || s == kZbH1) {
    if (v != 1) throw std::invalid_argument(name + " uses one chunk per rank (virtual_stages = 1)");
    const int warm = std::min(pp - rank - 1, m);
    int f = 0, b = 0;
    for (int i = 0; i < warm; ++i) acts.push_back({kF, f++, rank});
    while (f < m) {
      acts.push_back({kF, f++, rank});
      acts.push_back({kB, b++, rank});
    }
    while (b < m) acts.push_back({kB, b++, rank});
    return acts;
  }
  if (m % pp != 0) throw std::invalid_argument("interleaved_1f1b needs microbatches % pp == 0");
  const int total = m * v;
  auto fwd = [&](int k) { return Action{kF, (k / (pp * v)) * pp + k % pp, ((k / pp) % v) * pp + rank}; };
  auto bwd = [&](int k) { return Action{kB, (k / (pp * v)) * pp + k % pp, (v - 1 - (k / pp) % v) * pp + rank}; };
  const int warm = std::min((pp - rank - 1) * 2 + (v - 1) * pp, total);
  int f = 0, b = 0;
  for (int i = 0; i < warm; ++i) acts.push_back(fwd(f++));
  while (f < total) {
    acts.push_back(fwd(f++));
    acts.push_back(bwd(b++));
  }
  while (b < total) acts.push_back(bwd(b++));
  return acts;
}

std::vector<std::tuple<std::string, int, int>> py_make(const std::string& name, int pp, int rank, int m, int v) {
  std::vector<std::tuple<std::string, int, int>> out;
  for (const Action& a : make(name, pp, rank, m, v)) out.emplace_back(a.kind == kF ? "F" : "B", a.mb, a.chunk);
  return out;
}

double theoretical_bubble(const std::string& name, int p, int m, int v, double tf, double tb, double tw) {
  switch (parse(name)) {
    case kGpipe:
    case k1f1b:
      return static_cast<double>(p - 1) / (m + p - 1);
    case kInterleaved:
      return static_cast<double>(p - 1) / (static_cast<double>(v) * m + p - 1);
    default: {
      const double idle = (p - 1) * (tf + tb - tw);
      return idle / (m * (tf + tb + tw) + idle);
    }
  }
}

// Contiguous non-empty ranges minimising the largest range cost (dynamic programme over prefix sums).
std::vector<std::pair<int, int>> balance_partition(const std::vector<double>& costs, int parts) {
  const int n = static_cast<int>(costs.size());
  if (parts < 1 || parts > n) throw std::invalid_argument("balance_partition: 1 <= parts <= number of layers");
  std::vector<double> pre(static_cast<size_t>(n) + 1, 0.0);
  for (int i = 0; i < n; ++i) pre[static_cast<size_t>(i) + 1] = pre[static_cast<size_t>(i)] + costs[static_cast<size_t>(i)];
  const double inf = std::numeric_limits<double>::infinity();
  const size_t w = static_cast<size_t>(n) + 1;
  std::vector<double> best((static_cast<size_t>(parts) + 1) * w, inf);
  std::vector<int> cut((static_cast<size_t>(parts) + 1) * w, 0);
  best[0] = 0.0;
  for (int k = 1; k <= parts; ++k)
    for (int i = k; i <= n; ++i)
      for (int j = k - 1; j < i; ++j) {
        const double c = std::max(best[static_cast<size_t>(k - 1) * w + static_cast<size_t>(j)],
                                  pre[static_cast<size_t>(i)] - pre[static_cast<size_t>(j)]);
        if (c < best[static_cast<size_t>(k) * w + static_cast<size_t>(i)]) {
          best[static_cast<size_t>(k) * w + static_cast<size_t>(i)] = c;
          cut[static_cast<size_t>(k) * w + static_cast<size_t>(i)] = j;
        }
      }
  std::vector<std::pair<int, int>> out;
  int i = n;
  for (int k = parts; k >= 1; --k) {
    const int j = cut[static_cast<size_t>(k) * w + static_cast<size_t>(i)];
    out.emplace_back(j, i);
    i = j;
  }
  std::reverse(out.begin(), out.end());
  return out;
}

// Event-driven run of every rank's action list (transfers take no time); returns idle / total.  ZB-H1 splits the
// backward into B (input gradient) and W (weight gradient); W runs in the gaps, at most pp - rank of them deferred.
double simulate_bubble(const std::string& name, int pp, int m, int v, double tf, double tb, double tw) {
  const bool split = parse(name) == kZbH1;
  std::vector<std::vector<Action>> acts;
  for (int r = 0; r < pp; ++r) acts.push_back(make(name, pp, r, m, v));
  const int nchunks = pp * v;
  std::map<std::tuple<int, int, int>, double> done;
  std::vector<double> clock(static_cast<size_t>(pp), 0.0), busy(static_cast<size_t>(pp), 0.0);
  std::vector<size_t> ptr(static_cast<size_t>(pp), 0);
  std::vector<int> pending_w(static_cast<size_t>(pp), 0);
  bool progressed = true;
  while (progressed) {
    progressed = false;
    for (int r = 0; r < pp; ++r) {
      const size_t ri = static_cast<size_t>(r);
      while (ptr[ri] < acts[ri].size()) {
        const Action a = acts[ri][ptr[ri]];
        bool has_dep = true;
        std::tuple<int, int, int> dep;
        if (a.kind == kF) {
          if (a.chunk > 0) dep = {kF, a.mb, a.chunk - 1}; else has_dep = false;
        } else {
          dep = a.chunk < nchunks - 1 ? std::make_tuple(static_cast<int>(kB), a.mb, a.chunk + 1)
                                      : std::make_tuple(static_cast<int>(kF), a.mb, a.chunk);
        }
        double ready = 0.0;
        if (has_dep) {
          auto it = done.find(dep);
          if (it == done.end()) break;
          ready = it->second;
        }
        if (split) {
          while (pending_w[ri] > 0 && clock[ri] + tw <= ready + 1e-12) {
            --pending_w[ri];
            clock[ri] += tw;
            busy[ri] += tw;
          }
          while (pending_w[ri] > pp - r) {
            --pending_w[ri];
            clock[ri] += tw;
            busy[ri] += tw;
          }
        }
        const double start = std::max(clock[ri], ready);
        const double dur = a.kind == kF ? tf : (split ? tb : tb + tw);
        clock[ri] = start + dur;
        busy[ri] += dur;
        done[{a.kind, a.mb, a.chunk}] = clock[ri];
        if (split && a.kind == kB) ++pending_w[ri];
        ++ptr[ri];
        progressed = true;
      }
    }
  }
  double total = 0.0, work = 0.0;
  for (int r = 0; r < pp; ++r) {
    const size_t ri = static_cast<size_t>(r);
    clock[ri] += tw * pending_w[ri];
    busy[ri] += tw * pending_w[ri];
    total = std::max(total, clock[ri]);
    work += busy[ri];
  }
  return 1.0 - work / (total * pp);
}

}  // namespace

void bind_pipeline_sched(py::module_& m) {
  m.def("pipe_make_schedule", &py_make);
  m.def("pipe_theoretical_bubble", &theoretical_bubble);
  m.def("pipe_balance_partition", &balance_partition);
  m.def("pipe_simulate_bubble", &simulate_bubble);
}
