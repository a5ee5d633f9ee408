// Capacity assignment of the CPU mixture-of-experts core: which (token, choice) pairs an expert accepts, where their
// rows go in the expert-sorted buffer, and what happens to the overflow.
//   * tokens are split into `groups` equal groups; every expert takes at most `capacity` rows per group;
//   * inside a group the order is (choice j, token t): every first choice is served before any second choice;
//   * overflow "drop": the pair is dropped; "reroute": the pair goes to the token's best-ranked expert that the
//     token has not chosen and that still has room in this group, else it is dropped;
//   * rows are laid out expert by expert, inside an expert group by group, inside a group in assignment order
//     (a counting sort, so the layout is deterministic).
// Parity: the routing walk of src/moe/moe.cpp:115-259 in the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <vector>

namespace py = pybind11;

namespace {

using I64 = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

// expert [N, k]: chosen experts by rank; order [N, E]: every expert by descending score (only read when rerouting).
py::tuple moe_assign(const I64& expert_in, const I64& order, int experts, int groups, int64_t capacity, bool reroute) {
  if (expert_in.ndim() != 2) throw std::invalid_argument("moe_assign: expert must be [tokens, k]");
  const int64_t N = expert_in.shape(0), k = expert_in.shape(1);
  if (groups <= 0 || N % groups != 0) throw std::invalid_argument("moe_assign: tokens must divide by groups");
  if (experts <= 0 || capacity < 0) throw std::invalid_argument("moe_assign: bad experts / capacity");
  if (reroute && (order.ndim() != 2 || order.shape(0) != N || order.shape(1) != experts))
    throw std::invalid_argument("moe_assign: order must be [tokens, experts] when rerouting");
  const int64_t Ng = N / groups;
  py::array_t<int64_t> expert_out({N, k}), row({N, k}), offsets(static_cast<py::ssize_t>(experts) + 1);
  int64_t* ex = expert_out.mutable_data();
  int64_t* rw = row.mutable_data();
  int64_t* off = offsets.mutable_data();
  const int64_t* src = expert_in.data();
  const int64_t* ord = reroute ? order.data() : nullptr;
  for (int64_t i = 0; i < N * k; ++i) {
    if (src[i] < 0 || src[i] >= experts) throw std::out_of_range("moe_assign: expert index outside [0, experts)");
    ex[i] = src[i];
    rw[i] = -1;
  }
  // pass 1: acceptance; slot_in_group[t, j] = position among the rows expert e accepted in this group
  std::vector<int64_t> fill(static_cast<size_t>(groups) * experts, 0);     // [g][e] accepted rows
  std::vector<int64_t> within(static_cast<size_t>(N * k), -1);
  int64_t dropped = 0, rerouted = 0;
  for (int g = 0; g < groups; ++g) {
    int64_t* f = fill.data() + static_cast<size_t>(g) * experts;
    for (int64_t j = 0; j < k; ++j) {
      for (int64_t t = g * Ng; t < (g + 1) * Ng; ++t) {
        int64_t e = ex[t * k + j];
        if (f[e] >= capacity) {
          int64_t alt = -1;
          if (reroute) {
            for (int c = 0; c < experts && alt < 0; ++c) {
              const int64_t e2 = ord[t * experts + c];
              if (e2 < 0 || e2 >= experts) throw std::out_of_range("moe_assign: order holds a bad expert index");
              if (f[e2] >= capacity) continue;
              bool chosen = false;
              for (int64_t q = 0; q < k; ++q) chosen |= ex[t * k + q] == e2;
              if (!chosen) alt = e2;
            }
          }
          if (alt < 0) {
            ++dropped;
            continue;
          }
          ++rerouted;
          ex[t * k + j] = alt;
          e = alt;
        }
        within[static_cast<size_t>(t * k + j)] = f[e]++;
      }
    }
  }
  // pass 2: counting sort -> offsets per expert, base per (expert, group)
  std::vector<int64_t> base(static_cast<size_t>(groups) * experts, 0);
  int64_t next = 0;
  for (int e = 0; e < experts; ++e) {
    off[e] = next;
    for (int g = 0; g < groups; ++g) {
      base[static_cast<size_t>(g) * experts + e] = next;
      next += fill[static_cast<size_t>(g) * experts + e];
    }
  }
  off[experts] = next;
  py::array_t<int64_t> perm(next);
  int64_t* pt = perm.mutable_data();
  for (int64_t t = 0; t < N; ++t) {
    const int g = static_cast<int>(t / Ng);
    for (int64_t j = 0; j < k; ++j) {
      const int64_t w = within[static_cast<size_t>(t * k + j)];
      if (w < 0) continue;
      const int64_t r = base[static_cast<size_t>(g) * experts + ex[t * k + j]] + w;
      rw[t * k + j] = r;
      pt[r] = t;
    }
  }
  return py::make_tuple(expert_out, row, offsets, perm, dropped, rerouted);
}

}  // namespace

void bind_moe_route(py::module_& m) {
  m.def("moe_assign", &moe_assign, py::arg("expert"), py::arg("order"), py::arg("experts"), py::arg("groups"),
        py::arg("capacity"), py::arg("reroute"));
}
