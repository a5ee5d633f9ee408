// CPU forms of the fused training ops: cross-entropy with label smoothing and z-loss whose gradient overwrites the
// logits (no [rows, vocab] probability tensor is ever kept), and counter-based Philox dropout whose mask is a pure
// function of (seed, offset, element index).  Rows / blocks are split over worker threads; the loss is summed in
// double in row order, so the result does not depend on the number of threads.
//   loss_r = (1-s)(lse - x_t) + s(lse - mean x) + z lse^2          (valid rows; mean over valid rows)
//   g_rj   = (p_j (1 + 2 z lse) - s/V - (1-s)[j == t]) * scale / valid
// Parity: src/fused/training.cpp:53-135 (shifted CE) and :321-379 (Philox dropout) of the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

template <typename F>
void parallel_for(int64_t n, int64_t grain, F f) {
  const int64_t hw = std::max<int64_t>(1, std::thread::hardware_concurrency());
  const int64_t parts = std::max<int64_t>(1, std::min<int64_t>(hw, n / std::max<int64_t>(1, grain)));
  if (parts <= 1) {
    f(0, n);
    return;
  }
  std::vector<std::thread> th;
  th.reserve(static_cast<size_t>(parts));
  const int64_t step = (n + parts - 1) / parts;
  for (int64_t p = 0; p < parts; ++p) {
    const int64_t lo = p * step, hi = std::min(n, lo + step);
    if (lo >= hi) break;
    th.emplace_back([=, &f] { f(lo, hi); });
  }
  for (auto& t : th) t.join();
}

// logits [rows, ld] float32, rewritten with the gradient when write_grad; targets [rows] int32 (ignore_index or any
// value outside [0, vocab) other than ignore_index -> error).  Returns (mean loss, valid rows).
py::tuple cpu_cross_entropy(py::array_t<float, py::array::c_style> logits, py::array_t<int32_t, py::array::c_style> targets,
                            int vocab, int ignore_index, float smoothing, float z_loss, float grad_scale, bool write_grad) {
  if (logits.ndim() != 2 || targets.ndim() != 1 || targets.shape(0) != logits.shape(0))
    throw std::invalid_argument("cpu_cross_entropy: logits [rows, ld] and targets [rows] expected");
  const int64_t rows = logits.shape(0), ld = logits.shape(1);
  if (vocab <= 0 || vocab > ld) throw std::invalid_argument("cpu_cross_entropy: vocab must be in (0, ld]");
  float* x = logits.mutable_data();
  const int32_t* tg = targets.data();
  int64_t valid = 0;
  for (int64_t r = 0; r < rows; ++r) {
    if (tg[r] == ignore_index) continue;
    if (tg[r] < 0 || tg[r] >= vocab) throw std::out_of_range("cpu_cross_entropy: target outside the vocabulary");
    ++valid;
  }
  std::vector<double> row_loss(static_cast<size_t>(rows), 0.0);
  const float inv_valid = valid > 0 ? 1.0f / static_cast<float>(valid) : 0.0f;
  {
    py::gil_scoped_release nogil;
    parallel_for(rows, 8, [&](int64_t lo, int64_t hi) {
      for (int64_t r = lo; r < hi; ++r) {
        float* row = x + r * ld;
        if (tg[r] == ignore_index) {
          if (write_grad) std::fill(row, row + ld, 0.0f);
          continue;
        }
        float mx = row[0];
        double sum_x = 0.0;
        for (int j = 0; j < vocab; ++j) {
          mx = std::max(mx, row[j]);
          sum_x += row[j];
        }
        double se = 0.0;
        for (int j = 0; j < vocab; ++j) se += std::exp(static_cast<double>(row[j] - mx));
        const double lse = static_cast<double>(mx) + std::log(se);
        const double xt = row[tg[r]];
        row_loss[static_cast<size_t>(r)] =
            (1.0 - smoothing) * (lse - xt) + smoothing * (lse - sum_x / vocab) + static_cast<double>(z_loss) * lse * lse;
        if (!write_grad) continue;
        const float k = grad_scale * inv_valid;
        const float pz = static_cast<float>(1.0 + 2.0 * z_loss * lse) * k;
        const float sv = smoothing / static_cast<float>(vocab) * k;
        const float flse = static_cast<float>(lse);
        for (int j = 0; j < vocab; ++j) row[j] = std::exp(row[j] - flse) * pz - sv;
        row[tg[r]] -= (1.0f - smoothing) * k;
        std::fill(row + vocab, row + ld, 0.0f);          // padding columns carry no gradient
      }
    });
  }
  double total = 0.0;
  for (double v : row_loss) total += v;
  return py::make_tuple(valid > 0 ? total / static_cast<double>(valid) : 0.0, valid);
}

inline void philox10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = 0xD2511F53ull * c[0];
    const uint64_t p1 = 0xCD9E8D57ull * c[2];
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// y = keep ? x / (1 - p) : 0 with keep iff u >= p; element i uses counter block offset + i / 4, lane i % 4.
py::array_t<float> cpu_dropout_philox(py::array_t<float, py::array::c_style> x, float p, uint64_t seed, uint64_t offset) {
  if (!(p >= 0.0f && p < 1.0f)) throw std::invalid_argument("dropout probability must be in [0, 1)");
  std::vector<py::ssize_t> shape(x.shape(), x.shape() + x.ndim());
  py::array_t<float> out(shape);
  const float* src = x.data();
  float* dst = out.mutable_data();
  const int64_t n = x.size();
  const float scale = 1.0f / (1.0f - p);
  py::gil_scoped_release nogil;
  parallel_for((n + 3) / 4, 4096, [&](int64_t lo, int64_t hi) {
    for (int64_t b = lo; b < hi; ++b) {
      const uint64_t blk = offset + static_cast<uint64_t>(b);
      uint32_t c[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u};
      philox10(c, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
      for (int j = 0; j < 4 && b * 4 + j < n; ++j) {
        const float u = static_cast<float>(c[j] >> 8) * (1.0f / 16777216.0f);
        dst[b * 4 + j] = u >= p ? src[b * 4 + j] * scale : 0.0f;
      }
    }
  });
  return out;
}

}  // namespace

void bind_fused_train_cpu(py::module_& m) {
  m.def("cpu_cross_entropy", &cpu_cross_entropy, py::arg("logits"), py::arg("targets"), py::arg("vocab"),
        py::arg("ignore_index") = -100, py::arg("smoothing") = 0.0f, py::arg("z_loss") = 0.0f, py::arg("grad_scale") = 1.0f,
        py::arg("write_grad") = true);
  m.def("cpu_dropout_philox", &cpu_dropout_philox);
}
