// CPU oracles and host-side compute: Philox4x32-10, AdamW over a range with the exact device op
// order (no fused multiply-add; compile with -ffp-contract=off), FP64 squared norm in fixed
// chunks, FP64 math attention.
// Parity: include/nexus/cpu/adam.hpp + src/cpu/adam_avx2.cpp (bit-equal to the GPU update),
// src/fused/training.cpp:321-349 (Philox), include/nexus/attention/cpu.hpp (math_attention oracle).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

namespace py = pybind11;

namespace {

inline void philox_round(uint32_t c[4], uint32_t& k0, uint32_t& k1) {
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

py::array_t<float> philox_uniform(int64_t n, uint64_t seed, uint64_t offset) {
  py::array_t<float> out(n);
  float* o = out.mutable_data();
  for (int64_t b = 0; b * 4 < n; ++b) {
    const uint64_t blk = offset + static_cast<uint64_t>(b);
    uint32_t c[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u};
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
    for (int r = 0; r < 10; ++r) philox_round(c, k0, k1);
    for (int j = 0; j < 4 && b * 4 + j < n; ++j) o[b * 4 + j] = static_cast<float>(c[j] >> 8) * (1.0f / 16777216.0f);
  }
  return out;
}

// p, m, v updated in place; g read-only.  Returns nothing; the caller supplies the clip coefficient.
void adamw_range(py::array_t<float, py::array::c_style> p, py::array_t<float, py::array::c_style> g,
                 py::array_t<float, py::array::c_style> m, py::array_t<float, py::array::c_style> v, float lr,
                 float wd, float beta1, float beta2, float eps, float inv1, float inv2, float clip) {
  const int64_t n = p.size();
  if (g.size() != n || m.size() != n || v.size() != n) throw std::invalid_argument("adamw_range: size mismatch");
  float* pp = p.mutable_data();
  const float* gg = g.data();
  float* mm = m.mutable_data();
  float* vv = v.mutable_data();
  const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2, lrwd = lr * wd;
  for (int64_t i = 0; i < n; ++i) {
    const float gi = gg[i] * clip;
    float pi = pp[i];
    pi = pi - lrwd * pi;
    const float mi = beta1 * mm[i] + omb1 * gi;
    const float vi = beta2 * vv[i] + omb2 * (gi * gi);
    const float mh = mi * inv1;
    const float vh = vi * inv2;
    pi = pi - (lr * mh) / (std::sqrt(vh) + eps);
    pp[i] = pi;
    mm[i] = mi;
    vv[i] = vi;
  }
}

double sq_norm(py::array_t<float, py::array::c_style | py::array::forcecast> g) {
  const int64_t n = g.size();
  const float* p = g.data();
  constexpr int64_t kChunk = 1 << 20;  // fixed chunking: the result does not depend on threads
  double total = 0.0;
  for (int64_t b = 0; b < n; b += kChunk) {
    double acc = 0.0;
    const int64_t e = std::min(n, b + kChunk);
    for (int64_t i = b; i < e; ++i) acc += static_cast<double>(p[i]) * p[i];
    total += acc;
  }
  return total;
}

// q [B,Tq,H,D], k/v [B,Tk,Hkv,D] (double) -> o [B,Tq,H,D]; causal bottom-right aligned; window <= 0: none.
py::array_t<double> math_attention(py::array_t<double, py::array::c_style | py::array::forcecast> q,
                                   py::array_t<double, py::array::c_style | py::array::forcecast> k,
                                   py::array_t<double, py::array::c_style | py::array::forcecast> v, bool causal,
                                   int window, double scale, double softcap) {
  if (q.ndim() != 4 || k.ndim() != 4 || v.ndim() != 4) throw std::invalid_argument("math_attention: 4-D inputs");
  const int64_t B = q.shape(0), Tq = q.shape(1), H = q.shape(2), D = q.shape(3), Tk = k.shape(1), Hk = k.shape(2);
  if (H % Hk != 0) throw std::invalid_argument("math_attention: H % Hkv != 0");
  py::array_t<double> out({B, Tq, H, D});
  const double* Q = q.data();
  const double* K = k.data();
  const double* V = v.data();
  double* O = out.mutable_data();
  const int64_t off = Tk - Tq, grp = H / Hk;
  std::vector<double> s(static_cast<size_t>(Tk));
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < H; ++h)
      for (int64_t i = 0; i < Tq; ++i) {
        const double* qi = Q + ((b * Tq + i) * H + h) * D;
        double mx = -std::numeric_limits<double>::infinity();
        for (int64_t j = 0; j < Tk; ++j) {
          bool masked = (causal && j > i + off) || (window > 0 && j < i + off - window + 1);
          if (masked) {
            s[static_cast<size_t>(j)] = -std::numeric_limits<double>::infinity();
            continue;
          }
          const double* kj = K + ((b * Tk + j) * Hk + h / grp) * D;
          double d = 0.0;
          for (int64_t x = 0; x < D; ++x) d += qi[x] * kj[x];
          d *= scale;
          if (softcap > 0.0) d = softcap * std::tanh(d / softcap);
          s[static_cast<size_t>(j)] = d;
          mx = std::max(mx, d);
        }
        double* oi = O + ((b * Tq + i) * H + h) * D;
        for (int64_t x = 0; x < D; ++x) oi[x] = 0.0;
        if (!std::isfinite(mx)) continue;
        double sum = 0.0;
        for (int64_t j = 0; j < Tk; ++j) {
          const double e = std::isfinite(s[static_cast<size_t>(j)]) ? std::exp(s[static_cast<size_t>(j)] - mx) : 0.0;
          s[static_cast<size_t>(j)] = e;
          sum += e;
        }
        for (int64_t j = 0; j < Tk; ++j) {
          const double w = s[static_cast<size_t>(j)] / sum;
          if (w == 0.0) continue;
          const double* vj = V + ((b * Tk + j) * Hk + h / grp) * D;
          for (int64_t x = 0; x < D; ++x) oi[x] += w * vj[x];
        }
      }
  return out;
}

}  // namespace

void bind_cpu_kernels(py::module_& m) {
  m.def("philox_uniform", &philox_uniform);
  m.def("adamw_range", &adamw_range);
  m.def("sq_norm", &sq_norm);
  m.def("math_attention", &math_attention, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("causal") = true,
        py::arg("window") = 0, py::arg("scale") = 1.0, py::arg("softcap") = 0.0);
}
