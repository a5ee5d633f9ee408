// NXS3 durable checkpoint archive: named byte entries sealed by a SHA-256 of everything before it.
//   "NXS3\0\0\0\0" | u32 3 | u32 n | (u32 namelen | name | u64 bytes | data)* | 32-byte SHA-256
// Files are written to "<path>.part" and renamed, so a reader never sees a half-written archive.
// Parity: include/nexus/ckpt/checkpoint.hpp:8-28 and src/ckpt/{checkpoint,sha256}.cpp of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdio>
#include <fstream>

#include "bytes_io.hpp"
#include "sha256.hpp"

namespace py = pybind11;

namespace {

const char kMagic[8] = {'N', 'X', 'S', '3', 0, 0, 0, 0};

py::bytes nxs3_encode(const std::vector<std::pair<std::string, py::bytes>>& entries) {
  nxh::Writer w;
  w.raw(kMagic, 8);
  w.put<uint32_t>(3);
  w.put<uint32_t>(static_cast<uint32_t>(entries.size()));
  for (const auto& e : entries) {
    const std::string data = e.second;
    w.put<uint32_t>(static_cast<uint32_t>(e.first.size()));
    w.raw(e.first.data(), e.first.size());
    w.put<uint64_t>(data.size());
    w.raw(data.data(), data.size());
  }
  nxh::Sha256 sha;
  sha.update(w.buf.data(), w.buf.size());
  uint8_t digest[32];
  sha.finish(digest);
  w.raw(digest, 32);
  return py::bytes(reinterpret_cast<const char*>(w.buf.data()), w.buf.size());
}

py::list nxs3_decode(const py::bytes& blob) {
  const std::string s = blob;
  if (s.size() < 8 + 4 + 4 + 32) throw std::runtime_error("nxs3: file too short");
  const uint8_t* p = reinterpret_cast<const uint8_t*>(s.data());
  if (std::memcmp(p, kMagic, 8) != 0) throw std::runtime_error("nxs3: magic mismatch");
  nxh::Sha256 sha;
  sha.update(p, s.size() - 32);
  uint8_t digest[32];
  sha.finish(digest);
  if (std::memcmp(digest, p + s.size() - 32, 32) != 0) throw std::runtime_error("nxs3: checksum mismatch (corrupt file)");
  nxh::Reader r(p, s.size() - 32);
  r.raw(8);
  if (r.get<uint32_t>() != 3) throw std::runtime_error("nxs3: unsupported version");
  const uint32_t n = r.get<uint32_t>();
  py::list out;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t nl = r.get<uint32_t>();
    std::string name(reinterpret_cast<const char*>(r.raw(nl)), nl);
    const uint64_t bytes = r.get<uint64_t>();
    out.append(py::make_tuple(name, py::bytes(reinterpret_cast<const char*>(r.raw(bytes)), bytes)));
  }
  if (!r.done()) throw std::runtime_error("nxs3: trailing bytes before the checksum");
  return out;
}

std::string sha256_hex(const py::bytes& data) {
  const std::string s = data;
  nxh::Sha256 sha;
  sha.update(s.data(), s.size());
  uint8_t d[32];
  sha.finish(d);
  return nxh::Sha256::hex(d);
}

std::string sha256_file(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw std::runtime_error("cannot open " + path);
  nxh::Sha256 sha;
  std::vector<char> buf(1 << 20);
  while (in) {
    in.read(buf.data(), buf.size());
    if (in.gcount() > 0) sha.update(buf.data(), static_cast<size_t>(in.gcount()));
  }
  uint8_t d[32];
  sha.finish(d);
  return nxh::Sha256::hex(d);
}

// Atomic file write: "<path>.part" then rename.  `crash_before_rename` leaves the .part file behind
// (used by the crash-injection tests).
void write_file_atomic(const std::string& path, const py::bytes& data, bool crash_before_rename) {
  const std::string s = data;
  const std::string part = path + ".part";
  {
    std::ofstream out(part, std::ios::binary | std::ios::trunc);
    if (!out) throw std::runtime_error("cannot open " + part);
    out.write(s.data(), static_cast<std::streamsize>(s.size()));
    out.flush();
    if (!out) throw std::runtime_error("write failed: " + part);
  }
  if (crash_before_rename) return;
  if (std::rename(part.c_str(), path.c_str()) != 0) throw std::runtime_error("rename failed: " + path);
}

}  // namespace

void bind_nxs3(py::module_& m) {
  m.def("nxs3_encode", &nxs3_encode);
  m.def("nxs3_decode", &nxs3_decode);
  m.def("sha256_hex", &sha256_hex);
  m.def("sha256_file", &sha256_file);
  m.def("write_file_atomic", &write_file_atomic, py::arg("path"), py::arg("data"),
        py::arg("crash_before_rename") = false);
}
