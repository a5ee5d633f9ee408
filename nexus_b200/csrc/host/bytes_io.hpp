// Little-endian cursor over a byte buffer (reader) and an append-only byte sink (writer) used by the
// archive codecs.  Reads past the end throw "truncated".
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace nxh {

class Reader {
 public:
  Reader(const uint8_t* p, size_t n) : p_(p), n_(n) {}
  template <typename T>
  T get() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p_ + pos_, sizeof(T));
    pos_ += sizeof(T);
    return v;
  }
  std::string str() {
    const uint32_t len = get<uint32_t>();
    need(len);
    std::string s(reinterpret_cast<const char*>(p_ + pos_), len);
    pos_ += len;
    return s;
  }
  const uint8_t* raw(size_t len) {
    need(len);
    const uint8_t* q = p_ + pos_;
    pos_ += len;
    return q;
  }
  size_t pos() const { return pos_; }
  size_t size() const { return n_; }
  bool done() const { return pos_ == n_; }

 private:
  void need(size_t k) const {
    if (k > n_ - pos_) throw std::runtime_error("truncated archive");
  }
  const uint8_t* p_;
  size_t n_;
  size_t pos_ = 0;
};

class Writer {
 public:
  template <typename T>
  void put(T v) {
    const uint8_t* q = reinterpret_cast<const uint8_t*>(&v);
    buf.insert(buf.end(), q, q + sizeof(T));
  }
  void str(const std::string& s) {
    put<uint32_t>(static_cast<uint32_t>(s.size()));
    buf.insert(buf.end(), s.begin(), s.end());
  }
  void raw(const void* p, size_t n) {
    const uint8_t* q = static_cast<const uint8_t*>(p);
    buf.insert(buf.end(), q, q + n);
  }
  std::vector<uint8_t> buf;
};

}  // namespace nxh
