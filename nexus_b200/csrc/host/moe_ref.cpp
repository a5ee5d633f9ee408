// FP64 token-by-token oracle of the mixture-of-experts layer, independent of the tensor code it checks: router
// logits, stable top-k, gate = softmax over the selected logits, GShard capacity per token group with (choice, token)
// priority, Drop or Reroute overflow, SwiGLU experts, gate-weighted sum, auxiliary balance loss and router z-loss.
// Parity: the `reference()` oracle and the routing rules of src/moe/moe.cpp:94-259 of the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cmath>
#include <numeric>
#include <stdexcept>
#include <vector>

namespace py = pybind11;
using Arr = py::array_t<double, py::array::c_style | py::array::forcecast>;

namespace {

py::tuple moe_reference(Arr x_, Arr router_, Arr up_, Arr down_, int k, int groups, int capacity, bool reroute,
                        double aux_alpha, double z_alpha) {
  auto x = x_.unchecked<2>();            // [N, d]
  auto wg = router_.unchecked<2>();      // [d, E]
  auto up = up_.unchecked<3>();          // [E, 2F, d]
  auto down = down_.unchecked<3>();      // [E, d, F]
  const int N = static_cast<int>(x.shape(0)), d = static_cast<int>(x.shape(1)), E = static_cast<int>(wg.shape(1));
  const int F = static_cast<int>(up.shape(1)) / 2;
  if (wg.shape(0) != d || up.shape(0) != E || up.shape(2) != d || down.shape(0) != E || down.shape(1) != d ||
      down.shape(2) != F || k < 1 || k > E || groups < 1 || N % groups)
    throw std::invalid_argument("moe_reference: inconsistent shapes");
  const int Ng = N / groups;
  std::vector<std::vector<int>> order(N, std::vector<int>(E));
  std::vector<std::vector<int>> expert(N, std::vector<int>(k));
  std::vector<std::vector<double>> gate(N, std::vector<double>(k));
  std::vector<double> prob_sum(E, 0.0), routed(E, 0.0);
  double lse_sq = 0.0;
  std::vector<double> logits(E);
  for (int t = 0; t < N; ++t) {
    for (int e = 0; e < E; ++e) {
      double s = 0.0;
      for (int c = 0; c < d; ++c) s += x(t, c) * wg(c, e);
      logits[e] = s;
    }
    const double mx = *std::max_element(logits.begin(), logits.end());
    double se = 0.0;
    for (int e = 0; e < E; ++e) se += std::exp(logits[e] - mx);
    const double lse = mx + std::log(se);
    lse_sq += lse * lse;
    for (int e = 0; e < E; ++e) prob_sum[e] += std::exp(logits[e] - lse);
    std::iota(order[t].begin(), order[t].end(), 0);
    std::stable_sort(order[t].begin(), order[t].end(), [&](int a, int b) { return logits[a] > logits[b]; });
    double top = logits[order[t][0]], gs = 0.0;
    for (int j = 0; j < k; ++j) gs += std::exp(logits[order[t][j]] - top);
    for (int j = 0; j < k; ++j) {
      expert[t][j] = order[t][j];
      gate[t][j] = std::exp(logits[order[t][j]] - top) / gs;
      routed[order[t][j]] += 1.0;
    }
  }
  double aux = 0.0;
  for (int e = 0; e < E; ++e) aux += (routed[e] / (static_cast<double>(N) * k)) * (prob_sum[e] / N);
  aux *= aux_alpha * E;
  const double z = z_alpha * lse_sq / N;
  // capacity per group, every first choice before any second choice
  std::vector<std::vector<char>> keep(N, std::vector<char>(k, 0));
  long dropped = 0, rerouted = 0;
  for (int g = 0; g < groups; ++g) {
    std::vector<int> fill(E, 0);
    for (int j = 0; j < k; ++j)
      for (int t = g * Ng; t < (g + 1) * Ng; ++t) {
        int e = expert[t][j];
        if (fill[e] >= capacity) {
          int alt = -1;
          if (reroute)
            for (int cand : order[t]) {
              if (fill[cand] >= capacity) continue;
              if (std::find(expert[t].begin(), expert[t].end(), cand) != expert[t].end()) continue;
              alt = cand;
              break;
            }
          if (alt < 0) {
            ++dropped;
            continue;
          }
          ++rerouted;
          expert[t][j] = alt;
          e = alt;
        }
        ++fill[e];
        keep[t][j] = 1;
      }
  }
  Arr y_({N, d});
  auto y = y_.mutable_unchecked<2>();
  std::vector<double> h(2 * F), a(F);
  for (int t = 0; t < N; ++t) {
    for (int c = 0; c < d; ++c) y(t, c) = 0.0;
    for (int j = 0; j < k; ++j) {
      if (!keep[t][j]) continue;
      const int e = expert[t][j];
      for (int r = 0; r < 2 * F; ++r) {
        double s = 0.0;
        for (int c = 0; c < d; ++c) s += up(e, r, c) * x(t, c);
        h[r] = s;
      }
      for (int f = 0; f < F; ++f) a[f] = h[f] / (1.0 + std::exp(-h[f])) * h[F + f];
      for (int c = 0; c < d; ++c) {
        double s = 0.0;
        for (int f = 0; f < F; ++f) s += down(e, c, f) * a[f];
        y(t, c) += gate[t][j] * s;
      }
    }
  }
  return py::make_tuple(y_, aux, z, dropped, rerouted);
}

}  // namespace

void bind_moe_ref(py::module_& m) {
  m.def("moe_reference", &moe_reference, py::arg("x"), py::arg("router"), py::arg("up"), py::arg("down"), py::arg("k"),
        py::arg("groups"), py::arg("capacity"), py::arg("reroute"), py::arg("aux_alpha"), py::arg("z_alpha"),
        "FP64 token-by-token MoE oracle: (y [N, d], aux, z, dropped, rerouted)");
}
