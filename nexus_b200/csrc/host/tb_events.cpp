// TensorBoard event files without a protobuf library: CRC32C (Castagnoli, table-driven), the masked form TFRecord
// uses, the record framing (u64 length, masked CRC of the length, payload, masked CRC of the payload) and the
// hand-encoded `Event` message for a scalar summary or the file-version header.
//   Event { 1: double wall_time; 2: int64 step; 3: string file_version; 5: Summary { 1: Value { 1: tag; 2: float } } }
// Parity: include/nexus/train/loggers.hpp, src/train/loggers.cpp of the reference (event-file writer and reader).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <array>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace py = pybind11;

namespace {

const std::array<uint32_t, 256>& crc_table() {
  static const std::array<uint32_t, 256> table = [] {
    std::array<uint32_t, 256> t{};
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1u) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
      t[i] = c;
    }
    return t;
  }();
  return table;
}

uint32_t crc32c(const char* p, size_t n) {
  const auto& t = crc_table();
  uint32_t c = 0xFFFFFFFFu;
  for (size_t i = 0; i < n; ++i) c = t[(c ^ static_cast<uint8_t>(p[i])) & 0xFFu] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
uint32_t masked(uint32_t c) { return ((c >> 15) | (c << 17)) + 0xA282EAD8u; }

void put_varint(std::string& out, uint64_t n) {
  do {
    uint8_t b = n & 0x7Fu;
    n >>= 7;
    out.push_back(static_cast<char>(b | (n ? 0x80u : 0u)));
  } while (n);
}
void put_key(std::string& out, int field, int wire) { put_varint(out, static_cast<uint64_t>(field) << 3 | static_cast<uint64_t>(wire)); }
void put_bytes(std::string& out, int field, const std::string& payload) {
  put_key(out, field, 2);
  put_varint(out, payload.size());
  out += payload;
}
template <typename T>
void put_fixed(std::string& out, T v) {
  char b[sizeof(T)];
  std::memcpy(b, &v, sizeof(T));
  out.append(b, sizeof(T));
}

std::string event(double wall_time, int64_t step, const std::string& tag, bool has_value, float value, const std::string& file_version) {
  std::string msg;
  put_key(msg, 1, 1);
  put_fixed(msg, wall_time);
  put_key(msg, 2, 0);
  put_varint(msg, static_cast<uint64_t>(step));
  if (!file_version.empty()) put_bytes(msg, 3, file_version);
  if (has_value) {
    std::string val;
    put_bytes(val, 1, tag);
    put_key(val, 2, 5);
    put_fixed(val, value);
    std::string summary;
    put_bytes(summary, 1, val);
    put_bytes(msg, 5, summary);
  }
  return msg;
}

std::string frame(const std::string& payload) {
  std::string out;
  const uint64_t n = payload.size();
  put_fixed(out, n);
  put_fixed(out, masked(crc32c(out.data(), 8)));
  out += payload;
  put_fixed(out, masked(crc32c(payload.data(), payload.size())));
  return out;
}

struct Reader {
  const std::string& b;
  size_t i = 0, end;
  Reader(const std::string& s, size_t from, size_t to) : b(s), i(from), end(to) {}
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (i >= end) throw std::runtime_error("event file: truncated varint");
      const uint8_t c = static_cast<uint8_t>(b[i++]);
      v |= static_cast<uint64_t>(c & 0x7Fu) << shift;
      if (!(c & 0x80u)) return v;
    }
    throw std::runtime_error("event file: varint too long");
  }
  void need(size_t n) const {
    if (end - i < n) throw std::runtime_error("event file: truncated field");
  }
};

// Every scalar of an event file as (step, tag, value); both CRCs of every record are verified.
std::vector<std::tuple<int64_t, std::string, float>> read_scalars(const std::string& data) {
  std::vector<std::tuple<int64_t, std::string, float>> out;
  size_t pos = 0;
  while (pos < data.size()) {
    if (data.size() - pos < 12) throw std::runtime_error("event file: truncated record header");
    uint64_t len;
    uint32_t crc;
    std::memcpy(&len, data.data() + pos, 8);
    std::memcpy(&crc, data.data() + pos + 8, 4);
    if (crc != masked(crc32c(data.data() + pos, 8))) throw std::runtime_error("event file: length checksum differs");
    if (len > data.size() - pos - 12 || data.size() - pos - 12 - len < 4) throw std::runtime_error("event file: truncated record");
    const size_t body = pos + 12;
    std::memcpy(&crc, data.data() + body + len, 4);
    if (crc != masked(crc32c(data.data() + body, len))) throw std::runtime_error("event file: payload checksum differs");
    Reader ev(data, body, body + len);
    int64_t step = 0;
    while (ev.i < ev.end) {
      const uint64_t key = ev.varint();
      const int field = static_cast<int>(key >> 3), wire = static_cast<int>(key & 7);
      if (wire == 0) {
        const uint64_t v = ev.varint();
        if (field == 2) step = static_cast<int64_t>(v);
      } else if (wire == 1) {
        ev.need(8);
        ev.i += 8;
      } else if (wire == 5) {
        ev.need(4);
        ev.i += 4;
      } else if (wire == 2) {
        const uint64_t n = ev.varint();
        ev.need(n);
        if (field == 5) {                      // Summary: repeated Value
          Reader sm(data, ev.i, ev.i + n);
          while (sm.i < sm.end) {
            const uint64_t k2 = sm.varint();
            if ((k2 & 7) != 2) throw std::runtime_error("event file: unexpected field in a summary");
            const uint64_t n2 = sm.varint();
            sm.need(n2);
            if ((k2 >> 3) == 1) {
              Reader val(data, sm.i, sm.i + n2);
              std::string tag;
              float value = 0.0f;
              bool has = false;
              while (val.i < val.end) {
                const uint64_t k3 = val.varint();
                const int f3 = static_cast<int>(k3 >> 3), w3 = static_cast<int>(k3 & 7);
                if (w3 == 2) {
                  const uint64_t n3 = val.varint();
                  val.need(n3);
                  if (f3 == 1) tag.assign(data, val.i, n3);
                  val.i += n3;
                } else if (w3 == 5) {
                  val.need(4);
                  if (f3 == 2) {
                    std::memcpy(&value, data.data() + val.i, 4);
                    has = true;
                  }
                  val.i += 4;
                } else if (w3 == 0) {
                  val.varint();
                } else if (w3 == 1) {
                  val.need(8);
                  val.i += 8;
                } else {
                  throw std::runtime_error("event file: unsupported wire type");
                }
              }
              if (has) out.emplace_back(step, tag, value);
            }
            sm.i += n2;
          }
        }
        ev.i += n;
      } else {
        throw std::runtime_error("event file: unsupported wire type");
      }
    }
    pos = body + len + 4;
  }
  return out;
}

}  // namespace

void bind_tb_events(py::module_& m) {
  m.def("crc32c", [](const py::bytes& b) { std::string s = b; return crc32c(s.data(), s.size()); });
  m.def("masked_crc32c", [](const py::bytes& b) { std::string s = b; return masked(crc32c(s.data(), s.size())); });
  m.def("tb_scalar_record", [](double wall, int64_t step, const std::string& tag, float value) {
    return py::bytes(frame(event(wall, step, tag, true, value, "")));
  });
  m.def("tb_version_record", [](double wall, const std::string& version) {
    return py::bytes(frame(event(wall, 0, "", false, 0.0f, version)));
  });
  m.def("tb_read_scalars", [](const py::bytes& b) { return read_scalars(b); });
}
