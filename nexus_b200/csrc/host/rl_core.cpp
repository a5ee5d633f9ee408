// Reinforcement-learning host helpers: the sum tree behind proportional prioritised replay (set, batched set, stratified
// descent for a batch of draws) and generalised advantage estimation over one trajectory.
// Parity: PrioritizedReplayBuffer and gae of include/nexus/rl (buffers.hpp, ppo.hpp) in the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace py = pybind11;

namespace {

using DArr = py::array_t<double, py::array::c_style | py::array::forcecast>;
using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using IArr = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

class SumTree {
 public:
  explicit SumTree(int64_t capacity) {
    if (capacity <= 0) throw std::invalid_argument("SumTree: capacity must be positive");
    size_ = 1;
    while (size_ < capacity) size_ *= 2;
    tree_.assign(static_cast<size_t>(2 * size_), 0.0);
  }
  void set(int64_t i, double p) {
    if (i < 0 || i >= size_) throw std::out_of_range("SumTree: index outside the tree");
    if (!(p >= 0.0)) throw std::invalid_argument("SumTree: priorities are non-negative numbers");
    int64_t j = i + size_;
    tree_[static_cast<size_t>(j)] = p;
    for (j /= 2; j >= 1; j /= 2) tree_[static_cast<size_t>(j)] = tree_[static_cast<size_t>(2 * j)] + tree_[static_cast<size_t>(2 * j + 1)];
  }
  void set_many(const IArr& idx, const DArr& p) {
    if (idx.size() != p.size()) throw std::invalid_argument("SumTree: index and priority counts differ");
    for (py::ssize_t k = 0; k < idx.size(); ++k) set(idx.data()[k], p.data()[k]);
  }
  double total() const { return tree_[1]; }
  double get(int64_t i) const {
    if (i < 0 || i >= size_) throw std::out_of_range("SumTree: index outside the tree");
    return tree_[static_cast<size_t>(i + size_)];
  }
  int64_t leaves() const { return size_; }
  // Leaf whose cumulative-priority interval holds x (empty right subtrees are never entered).
  int64_t find(double x) const {
    int64_t j = 1;
    while (j < size_) {
      const double left = tree_[static_cast<size_t>(2 * j)], right = tree_[static_cast<size_t>(2 * j + 1)];
      if (x <= left || right <= 0.0) {
        j = 2 * j;
      } else {
        x -= left;
        j = 2 * j + 1;
      }
    }
    return j - size_;
  }
  // One descent per draw; `filled` caps the result at the last written slot.  Returns (indices, priorities).
  py::tuple sample(const DArr& draws, int64_t filled) const {
    const py::ssize_t n = draws.size();
    py::array_t<int64_t> idx(n);
    py::array_t<double> pr(n);
    for (py::ssize_t b = 0; b < n; ++b) {
      const int64_t i = std::min<int64_t>(find(draws.data()[b]), std::max<int64_t>(filled, 1) - 1);
      idx.mutable_data()[b] = i;
      pr.mutable_data()[b] = tree_[static_cast<size_t>(i + size_)];
    }
    return py::make_tuple(idx, pr);
  }

 private:
  int64_t size_ = 1;
  std::vector<double> tree_;
};

// adv_t = delta_t + gamma lam (1 - done_t) adv_{t+1},  delta_t = r_t + gamma V_{t+1} (1 - done_t) - V_t; returns adv + V.
py::tuple gae(const DArr& rewards, const DArr& values, const py::array_t<bool, py::array::c_style | py::array::forcecast>& dones,
              double last_value, double gamma, double lam) {
  const py::ssize_t T = rewards.size();
  if (values.size() != T || dones.size() != T) throw std::invalid_argument("gae: rewards, values and dones differ in length");
  py::array_t<float> adv(T), ret(T);
  double run = 0.0;
  for (py::ssize_t t = T - 1; t >= 0; --t) {
    const double nv = t == T - 1 ? last_value : values.data()[t + 1];
    const double nonterm = dones.data()[t] ? 0.0 : 1.0;
    const double delta = rewards.data()[t] + gamma * nv * nonterm - values.data()[t];
    run = delta + gamma * lam * nonterm * run;
    adv.mutable_data()[t] = static_cast<float>(run);
    ret.mutable_data()[t] = static_cast<float>(run) + static_cast<float>(values.data()[t]);
  }
  return py::make_tuple(adv, ret);
}

}  // namespace

void bind_rl_core(py::module_& m) {
  py::class_<SumTree>(m, "SumTree")
      .def(py::init<int64_t>())
      .def("set", &SumTree::set)
      .def("set_many", &SumTree::set_many)
      .def("get", &SumTree::get)
      .def("total", &SumTree::total)
      .def("leaves", &SumTree::leaves)
      .def("find", &SumTree::find)
      .def("sample", &SumTree::sample);
  m.def("gae", &gae, py::arg("rewards"), py::arg("values"), py::arg("dones"), py::arg("last_value"), py::arg("gamma") = 0.99,
        py::arg("lam") = 0.95);
}
