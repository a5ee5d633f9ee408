// NXS2 single-file model archive codec (network + weights + optimizer + trainer + RL + python payload).
//
// Wire format, little-endian:
//   "NXS2" | u16 version = 1 | u16 flags (1 optimizer, 2 trainer, 4 rl, 8 python)
//   u32 n_layers | LayerSpec*       LayerSpec = u16 type | str name | u32 n_attr | Attr* | u32 n_child | LayerSpec*
//                                   Attr = u8 kind (1 i32, 2 f32, 3 bool, 4 string) | str key | value
//                                   str = u32 len | bytes
//   u32 n_weights | (str name | u32 rank | u64 dims[rank] | u64 n | f32 values[n])*
//   [optimizer] "NXO1" | str algorithm | u64 step | u32 n | f64 lr[n] | u32 n_blob | (u64 len | bytes)* | u32 n | f64 scalars[n]
//   [trainer]   "NXS1" | u32 epoch | u32 global_step | f64 loss | f64 best | u8 stop | u32 n | (str | f64)*
//   [rl]        str kind | u32 n | Attr* | u32 n_net | (str name | u32 n | u32 sizes[n] | u64 adam_step | floats | floats)*
//               | u32 n | f32 elos[n] | u32 n | floats*            floats = u64 n | f32[n]
//   [python]    u64 n (<= 32 MiB) | bytes
// A file that starts with "NXS1" is a trainer-only record and is rejected as a model archive.
//
// Parity: include/nexus/model/nxs_format.hpp:26-233 and src/model/nxs.cpp:110-373,535-636 of the reference.
// The Python side sees plain dicts / lists / bytes / numpy arrays.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bytes_io.hpp"

namespace py = pybind11;
using nxh::Reader;
using nxh::Writer;

namespace {

constexpr uint16_t kOptim = 1, kTrainer = 2, kRl = 4, kPython = 8;
constexpr uint64_t kMaxPython = 32ull * 1024ull * 1024ull;

void write_attr(Writer& w, const py::handle& attr) {
  py::tuple t = py::cast<py::tuple>(attr);  // (key, kind, value)
  const std::string key = py::cast<std::string>(t[0]);
  const int kind = py::cast<int>(t[1]);
  w.put<uint8_t>(static_cast<uint8_t>(kind));
  w.str(key);
  switch (kind) {
    case 1: w.put<int32_t>(py::cast<int32_t>(t[2])); break;
    case 2: w.put<float>(py::cast<float>(t[2])); break;
    case 3: w.put<uint8_t>(py::cast<bool>(t[2]) ? 1 : 0); break;
    case 4: w.str(py::cast<std::string>(t[2])); break;
    default: throw std::runtime_error("nxs: unknown attribute kind");
  }
}

py::tuple read_attr(Reader& r) {
  const int kind = r.get<uint8_t>();
  const std::string key = r.str();
  switch (kind) {
    case 1: return py::make_tuple(key, kind, r.get<int32_t>());
    case 2: return py::make_tuple(key, kind, r.get<float>());
    case 3: return py::make_tuple(key, kind, r.get<uint8_t>() != 0);
    case 4: return py::make_tuple(key, kind, r.str());
    default: throw std::runtime_error("nxs: unknown attribute kind");
  }
}

void write_layer(Writer& w, const py::dict& spec, int depth = 0) {
  if (depth > 64) throw std::runtime_error("nxs: layer tree too deep");
  w.put<uint16_t>(py::cast<uint16_t>(spec["type"]));
  w.str(py::cast<std::string>(spec["name"]));
  py::list attrs = spec.contains("attrs") ? py::cast<py::list>(spec["attrs"]) : py::list();
  w.put<uint32_t>(static_cast<uint32_t>(attrs.size()));
  for (auto a : attrs) write_attr(w, a);
  py::list children = spec.contains("children") ? py::cast<py::list>(spec["children"]) : py::list();
  w.put<uint32_t>(static_cast<uint32_t>(children.size()));
  for (auto c : children) write_layer(w, py::cast<py::dict>(c), depth + 1);
}

py::dict read_layer(Reader& r, int depth = 0) {
  if (depth > 64) throw std::runtime_error("nxs: layer tree too deep");
  py::dict spec;
  spec["type"] = r.get<uint16_t>();
  spec["name"] = r.str();
  const uint32_t na = r.get<uint32_t>();
  py::list attrs;
  for (uint32_t i = 0; i < na; ++i) attrs.append(read_attr(r));
  spec["attrs"] = attrs;
  const uint32_t nc = r.get<uint32_t>();
  py::list children;
  for (uint32_t i = 0; i < nc; ++i) children.append(read_layer(r, depth + 1));
  spec["children"] = children;
  return spec;
}

void write_floats(Writer& w, const py::handle& h) {
  auto arr = py::array_t<float, py::array::c_style | py::array::forcecast>::ensure(h);
  if (!arr) throw std::runtime_error("nxs: expected a float array");
  w.put<uint64_t>(static_cast<uint64_t>(arr.size()));
  w.raw(arr.data(), static_cast<size_t>(arr.size()) * sizeof(float));
}

py::array_t<float> read_floats(Reader& r) {
  const uint64_t n = r.get<uint64_t>();
  if (n > r.size() / sizeof(float)) throw std::runtime_error("truncated archive");
  py::array_t<float> out(static_cast<py::ssize_t>(n));
  if (n) std::memcpy(out.mutable_data(), r.raw(n * sizeof(float)), n * sizeof(float));
  return out;
}

py::bytes encode(const py::dict& archive) {
  Writer w;
  w.raw("NXS2", 4);
  w.put<uint16_t>(1);
  const bool has_optim = archive.contains("optim") && !archive["optim"].is_none();
  const bool has_trainer = archive.contains("trainer") && !archive["trainer"].is_none();
  const bool has_rl = archive.contains("rl") && !archive["rl"].is_none();
  std::string python;
  if (archive.contains("python") && !archive["python"].is_none()) python = py::cast<std::string>(archive["python"]);
  if (python.size() > kMaxPython) throw std::runtime_error("nxs python payload is too large");
  uint16_t flags = 0;
  if (has_optim) flags |= kOptim;
  if (has_trainer) flags |= kTrainer;
  if (has_rl) flags |= kRl;
  if (!python.empty()) flags |= kPython;
  w.put<uint16_t>(flags);
  py::list layers = py::cast<py::list>(archive["layers"]);
  w.put<uint32_t>(static_cast<uint32_t>(layers.size()));
  for (auto l : layers) write_layer(w, py::cast<py::dict>(l));
  py::list weights = archive.contains("weights") ? py::cast<py::list>(archive["weights"]) : py::list();
  w.put<uint32_t>(static_cast<uint32_t>(weights.size()));
  for (auto item : weights) {
    py::tuple t = py::cast<py::tuple>(item);  // (name, dims, values)
    w.str(py::cast<std::string>(t[0]));
    std::vector<uint64_t> dims = py::cast<std::vector<uint64_t>>(t[1]);
    w.put<uint32_t>(static_cast<uint32_t>(dims.size()));
    for (uint64_t d : dims) w.put<uint64_t>(d);
    write_floats(w, t[2]);
  }
  if (has_optim) {
    py::dict o = py::cast<py::dict>(archive["optim"]);
    w.raw("NXO1", 4);
    w.str(py::cast<std::string>(o["algorithm"]));
    w.put<uint64_t>(py::cast<uint64_t>(o["step"]));
    std::vector<double> lr = py::cast<std::vector<double>>(o["lr"]);
    w.put<uint32_t>(static_cast<uint32_t>(lr.size()));
    for (double v : lr) w.put<double>(v);
    py::list blobs = py::cast<py::list>(o["blobs"]);
    w.put<uint32_t>(static_cast<uint32_t>(blobs.size()));
    for (auto b : blobs) {
      const std::string s = py::cast<std::string>(b);
      w.put<uint64_t>(s.size());
      w.raw(s.data(), s.size());
    }
    std::vector<double> sc = py::cast<std::vector<double>>(o["scalars"]);
    w.put<uint32_t>(static_cast<uint32_t>(sc.size()));
    for (double v : sc) w.put<double>(v);
  }
  if (has_trainer) {
    py::dict t = py::cast<py::dict>(archive["trainer"]);
    w.raw("NXS1", 4);
    w.put<uint32_t>(py::cast<uint32_t>(t["epoch"]));
    w.put<uint32_t>(py::cast<uint32_t>(t["global_step"]));
    w.put<double>(py::cast<double>(t["loss"]));
    w.put<double>(py::cast<double>(t["best"]));
    w.put<uint8_t>(py::cast<bool>(t["stop"]) ? 1 : 0);
    py::list metrics = py::cast<py::list>(t["metrics"]);
    w.put<uint32_t>(static_cast<uint32_t>(metrics.size()));
    for (auto m : metrics) {
      py::tuple mt = py::cast<py::tuple>(m);
      w.str(py::cast<std::string>(mt[0]));
      w.put<double>(py::cast<double>(mt[1]));
    }
  }
  if (has_rl) {
    py::dict rl = py::cast<py::dict>(archive["rl"]);
    w.str(py::cast<std::string>(rl["kind"]));
    py::list cfg = py::cast<py::list>(rl["config"]);
    w.put<uint32_t>(static_cast<uint32_t>(cfg.size()));
    for (auto a : cfg) write_attr(w, a);
    py::list nets = py::cast<py::list>(rl["nets"]);
    w.put<uint32_t>(static_cast<uint32_t>(nets.size()));
    for (auto n : nets) {
      py::dict nd = py::cast<py::dict>(n);
      w.str(py::cast<std::string>(nd["name"]));
      std::vector<uint32_t> sizes = py::cast<std::vector<uint32_t>>(nd["sizes"]);
      w.put<uint32_t>(static_cast<uint32_t>(sizes.size()));
      for (uint32_t s : sizes) w.put<uint32_t>(s);
      w.put<uint64_t>(py::cast<uint64_t>(nd["adam_step"]));
      write_floats(w, nd["parameters"]);
      write_floats(w, nd["moments"]);
    }
    std::vector<float> elos = py::cast<std::vector<float>>(rl["elos"]);
    w.put<uint32_t>(static_cast<uint32_t>(elos.size()));
    for (float e : elos) w.put<float>(e);
    py::list pw = py::cast<py::list>(rl["player_weights"]);
    w.put<uint32_t>(static_cast<uint32_t>(pw.size()));
    for (auto p : pw) write_floats(w, p);
  }
  if (!python.empty()) {
    w.put<uint64_t>(python.size());
    w.raw(python.data(), python.size());
  }
  return py::bytes(reinterpret_cast<const char*>(w.buf.data()), w.buf.size());
}

py::dict decode(const py::bytes& data) {
  std::string s = data;
  Reader r(reinterpret_cast<const uint8_t*>(s.data()), s.size());
  const uint8_t* magic = r.raw(4);
  if (std::memcmp(magic, "NXS1", 4) == 0) throw std::runtime_error("this is a trainer state record, not a model archive");
  if (std::memcmp(magic, "NXS2", 4) != 0) throw std::runtime_error("nxs magic mismatch");
  if (r.get<uint16_t>() != 1) throw std::runtime_error("nxs version is unsupported");
  const uint16_t flags = r.get<uint16_t>();
  py::dict out;
  out["version"] = 1;
  const uint32_t nl = r.get<uint32_t>();
  py::list layers;
  for (uint32_t i = 0; i < nl; ++i) layers.append(read_layer(r));
  out["layers"] = layers;
  const uint32_t nw = r.get<uint32_t>();
  py::list weights;
  for (uint32_t i = 0; i < nw; ++i) {
    const std::string name = r.str();
    const uint32_t rank = r.get<uint32_t>();
    if (rank > 16) throw std::runtime_error("nxs: weight rank is implausible");
    std::vector<uint64_t> dims(rank);
    for (auto& d : dims) d = r.get<uint64_t>();
    weights.append(py::make_tuple(name, dims, read_floats(r)));
  }
  out["weights"] = weights;
  out["optim"] = py::none();
  out["trainer"] = py::none();
  out["rl"] = py::none();
  out["python"] = py::none();
  if (flags & kOptim) {
    if (std::memcmp(r.raw(4), "NXO1", 4) != 0) throw std::runtime_error("nxs optimizer magic mismatch");
    py::dict o;
    o["algorithm"] = r.str();
    o["step"] = r.get<uint64_t>();
    std::vector<double> lr(r.get<uint32_t>());
    for (auto& v : lr) v = r.get<double>();
    o["lr"] = lr;
    py::list blobs;
    const uint32_t nb = r.get<uint32_t>();
    for (uint32_t i = 0; i < nb; ++i) {
      const uint64_t len = r.get<uint64_t>();
      blobs.append(py::bytes(reinterpret_cast<const char*>(r.raw(len)), len));
    }
    o["blobs"] = blobs;
    std::vector<double> sc(r.get<uint32_t>());
    for (auto& v : sc) v = r.get<double>();
    o["scalars"] = sc;
    out["optim"] = o;
  }
  if (flags & kTrainer) {
    if (std::memcmp(r.raw(4), "NXS1", 4) != 0) throw std::runtime_error("nxs trainer magic mismatch");
    py::dict t;
    t["epoch"] = r.get<uint32_t>();
    t["global_step"] = r.get<uint32_t>();
    t["loss"] = r.get<double>();
    t["best"] = r.get<double>();
    t["stop"] = r.get<uint8_t>() != 0;
    py::list metrics;
    const uint32_t n = r.get<uint32_t>();
    for (uint32_t i = 0; i < n; ++i) {
      std::string name = r.str();
      metrics.append(py::make_tuple(name, r.get<double>()));
    }
    t["metrics"] = metrics;
    out["trainer"] = t;
  }
  if (flags & kRl) {
    py::dict rl;
    rl["kind"] = r.str();
    py::list cfg;
    const uint32_t na = r.get<uint32_t>();
    for (uint32_t i = 0; i < na; ++i) cfg.append(read_attr(r));
    rl["config"] = cfg;
    py::list nets;
    const uint32_t nn = r.get<uint32_t>();
    for (uint32_t i = 0; i < nn; ++i) {
      py::dict nd;
      nd["name"] = r.str();
      std::vector<uint32_t> sizes(r.get<uint32_t>());
      for (auto& v : sizes) v = r.get<uint32_t>();
      nd["sizes"] = sizes;
      nd["adam_step"] = r.get<uint64_t>();
      nd["parameters"] = read_floats(r);
      nd["moments"] = read_floats(r);
      nets.append(nd);
    }
    rl["nets"] = nets;
    std::vector<float> elos(r.get<uint32_t>());
    for (auto& v : elos) v = r.get<float>();
    rl["elos"] = elos;
    py::list pw;
    const uint32_t np_ = r.get<uint32_t>();
    for (uint32_t i = 0; i < np_; ++i) pw.append(read_floats(r));
    rl["player_weights"] = pw;
    out["rl"] = rl;
  }
  if (flags & kPython) {
    const uint64_t n = r.get<uint64_t>();
    if (n > kMaxPython) throw std::runtime_error("nxs python payload is too large");
    out["python"] = py::bytes(reinterpret_cast<const char*>(r.raw(n)), n);
  }
  return out;
}

}  // namespace

void bind_nxs2(py::module_& m) {
  m.def("nxs2_encode", &encode, "Serialise an archive dict to NXS2 bytes");
  m.def("nxs2_decode", &decode, "Parse NXS2 bytes into an archive dict");
}
