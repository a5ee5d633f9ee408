// Host-side low-precision number formats: float32 <-> bfloat16 / float16 / FP8 (E4M3fn, E5M2) bit patterns, all with
// round-to-nearest-even, written at the bit level (no compiler half types), plus the dtype promotion table.
// FP8 encode saturates to the largest finite value (E4M3fn has no infinity; E5M2's infinities are never produced) and
// maps NaN to the format's NaN code.
// Parity: include/nexus/core/half.hpp, include/nexus/core/fp8.hpp, include/nexus/core/dtype.hpp of the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace py = pybind11;

namespace {

inline uint32_t bits_of(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float float_of(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline uint16_t f32_to_bf16(float f) {
  const uint32_t u = bits_of(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0;
  return static_cast<uint16_t>((u + (0x7FFFu + ((u >> 16) & 1u))) >> 16);
}
inline float bf16_to_f32(uint16_t b) { return float_of(static_cast<uint32_t>(b) << 16); }

// Generic IEEE-like narrow float: `E` exponent bits, `M` mantissa bits.  `finite_only`: the all-ones exponent is an
// ordinary binade except for the all-ones mantissa (E4M3fn).  Overflow: `saturate` -> largest finite, else infinity.
template <int E, int M, bool FiniteOnly, bool Saturate>
inline uint32_t encode_small(float f) {
  constexpr int bias = (1 << (E - 1)) - 1;
  constexpr uint32_t exp_all = (1u << E) - 1;
  constexpr uint32_t max_code = FiniteOnly ? ((exp_all << M) | ((1u << M) - 2)) : (((exp_all - 1) << M) | ((1u << M) - 1));
  constexpr uint32_t inf_code = exp_all << M;
  constexpr uint32_t nan_code = FiniteOnly ? ((exp_all << M) | ((1u << M) - 1)) : ((exp_all << M) | (1u << (M - 1)));
  const uint32_t u = bits_of(f);
  const uint32_t sign = (u >> 31) << (E + M);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (E == 5 && M == 10) ? (sign | nan_code) : nan_code;   // FP8: one NaN code, sign dropped
  if (a == 0x7F800000u) return sign | (Saturate ? max_code : inf_code);
  const int e32 = static_cast<int>(a >> 23) - 127;
  uint32_t man = (a & 0x7FFFFFu) | (a >= 0x00800000u ? 0x800000u : 0u);     // 24-bit significand (implicit one)
  int e = e32;
  if (a < 0x00800000u) e = -126;                                            // float32 subnormal: no implicit one
  // target: value = man * 2^(e - 23); normal target exponent field = e + bias (>= 1), mantissa keeps M bits
  int shift = 23 - M;                                                       // bits to drop for a normal result
  int field = e + bias;
  if (field < 1) {                                                          // subnormal in the target format
    shift += 1 - field;
    field = 0;
  }
  uint32_t q;
  if (shift > 31) {
    q = 0;
  } else {
    const uint32_t drop = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    q = man >> shift;
    if (drop > half || (drop == half && (q & 1u))) ++q;
  }
  // q holds the implicit one for normals: q in [2^M, 2^(M+1)]; subnormals: q in [0, 2^M]
  uint32_t code;
  if (field == 0) {
    code = q;                                // q == 2^M rolls into the first normal: exponent field 1, mantissa 0
  } else {
    code = (static_cast<uint32_t>(field) << M) + (q - (1u << M));   // a carry out of the mantissa bumps the exponent
  }
  const uint32_t limit = max_code;
  if (code > limit) code = Saturate ? max_code : inf_code;
  return sign | code;
}

template <int E, int M, bool FiniteOnly>
inline float decode_small(uint32_t code) {
  constexpr int bias = (1 << (E - 1)) - 1;
  constexpr uint32_t exp_all = (1u << E) - 1;
  const bool neg = (code >> (E + M)) & 1u;
  const uint32_t e = (code >> M) & exp_all, m = code & ((1u << M) - 1);
  float v;
  if (FiniteOnly) {
    if (e == exp_all && m == (1u << M) - 1) return std::nanf("");
  } else if (e == exp_all) {
    if (m != 0) return std::nanf("");
    return neg ? -INFINITY : INFINITY;
  }
  if (e == 0) v = std::ldexp(static_cast<float>(m), 1 - bias - M);
  else v = std::ldexp(1.0f + static_cast<float>(m) / static_cast<float>(1u << M), static_cast<int>(e) - bias);
  return neg ? -v : v;
}

using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using U16Arr = py::array_t<uint16_t, py::array::c_style | py::array::forcecast>;
using U8Arr = py::array_t<uint8_t, py::array::c_style | py::array::forcecast>;

template <typename Out, typename In, typename F>
py::array_t<Out> map_array(const py::array_t<In, py::array::c_style | py::array::forcecast>& in, F f) {
  std::vector<py::ssize_t> shape(in.shape(), in.shape() + in.ndim());
  py::array_t<Out> out(shape);
  const In* src = in.data();
  Out* dst = out.mutable_data();
  const py::ssize_t n = in.size();
  for (py::ssize_t i = 0; i < n; ++i) dst[i] = f(src[i]);
  return out;
}

// DType ids follow the framework's enum: F32 0, F16 1, BF16 2, F64 3, I32 4, I64 5, I8 6, U8 7, Bool 8, F8E4M3 9, F8E5M2 10.
enum : int { F32, F16, BF16, F64, I32, I64, I8, U8, Bool, F8E4M3, F8E5M2, kCount };

int float_rank(int d) { return d == F16 || d == BF16 ? 1 : d == F32 ? 2 : d == F64 ? 3 : 0; }
int int_rank(int d) { return d == U8 ? 1 : d == I8 ? 2 : d == I32 ? 3 : d == I64 ? 4 : 0; }

int promote(int a, int b) {
  if (a < 0 || a >= kCount || b < 0 || b >= kCount) throw std::invalid_argument("promote: unknown dtype");
  if (a == b) return a;
  if (a >= F8E4M3 || b >= F8E4M3) throw std::domain_error("FP8 does not promote implicitly; convert FP8 explicitly");
  if (a == Bool) return b;
  if (b == Bool) return a;
  const int fa = float_rank(a), fb = float_rank(b);
  if ((fa != 0) != (fb != 0)) return fa != 0 ? a : b;
  if (fa != 0) {
    if (fa == fb) return F32;                          // F16 + BF16
    return fa > fb ? a : b;
  }
  if ((a == U8 && b == I8) || (a == I8 && b == U8)) return I32;   // documented deviation: PyTorch gives int16
  return int_rank(a) >= int_rank(b) ? a : b;
}

}  // namespace

void bind_lowp(py::module_& m) {
  m.def("f32_to_bf16_bits", [](const FArr& x) { return map_array<uint16_t, float>(x, f32_to_bf16); });
  m.def("bf16_bits_to_f32", [](const U16Arr& x) { return map_array<float, uint16_t>(x, bf16_to_f32); });
  m.def("f32_to_f16_bits", [](const FArr& x) {
    return map_array<uint16_t, float>(x, [](float f) { return static_cast<uint16_t>(encode_small<5, 10, false, false>(f)); });
  });
  m.def("f16_bits_to_f32", [](const U16Arr& x) {
    return map_array<float, uint16_t>(x, [](uint16_t c) { return decode_small<5, 10, false>(c); });
  });
  m.def("f32_to_fp8_bits", [](const FArr& x, bool e5m2) {
    if (e5m2) return map_array<uint8_t, float>(x, [](float f) { return static_cast<uint8_t>(encode_small<5, 2, false, true>(f)); });
    return map_array<uint8_t, float>(x, [](float f) { return static_cast<uint8_t>(encode_small<4, 3, true, true>(f)); });
  }, py::arg("x"), py::arg("e5m2") = false);
  m.def("fp8_bits_to_f32", [](const U8Arr& x, bool e5m2) {
    if (e5m2) return map_array<float, uint8_t>(x, [](uint8_t c) { return decode_small<5, 2, false>(c); });
    return map_array<float, uint8_t>(x, [](uint8_t c) { return decode_small<4, 3, true>(c); });
  }, py::arg("codes"), py::arg("e5m2") = false);
  m.def("dtype_promote", &promote);
}
