// Memory-mapped token shards with a prefetching reader thread.
//
// A shard is the tokenizer tool's file: "NXTK", u32 version (1), u32 vocabulary, u64 count, then `count` tokens as
// u16 (vocabulary <= 65536) or u32.  A reader maps any number of shards, cuts each into windows of `seq_len` tokens
// (a shard's ragged tail is dropped) and numbers the windows across shards.  Rows are handed out by a global cursor:
// row g of the job reads window perm(g / total, g % total); rank r of w takes g = cursor * w + r, so ranks read disjoint
// rows and the cursor alone describes the position (resume and a change of the rank count need nothing else).  The
// per-epoch permutation is a keyed Feistel network over the next power of four with cycle walking: a bijection on
// [0, total) with no table, so a job can jump to any cursor in O(1).  A worker thread keeps `depth` batches decoded to
// int32 ahead of the consumer; calls wait without the interpreter lock.
// Parity: the token loader of include/nexus/cuda/token_loader.hpp and the TokenBatchSource contract
// (next / state / restore / global cursor) of include/nexus/train/lm_trainer.hpp in the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

struct Shard {
  std::string path;
  const uint8_t* base = nullptr;   // mapping
  size_t bytes = 0;
  const uint8_t* data = nullptr;   // first token
  uint64_t count = 0;
  uint32_t vocab = 0;
  int width = 2;                   // bytes per token
  uint64_t first_window = 0, windows = 0;
};

uint64_t mix64(uint64_t x) {       // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Bijection on [0, n): four Feistel rounds on 2*half bits, re-applied while the image falls outside [0, n).
uint64_t permute(uint64_t i, uint64_t n, uint64_t key) {
  if (n <= 1) return 0;
  if (n > (1ull << 60)) throw std::invalid_argument("permute: domain too large");
  int half = 1;
  while ((1ull << (2 * half)) < n) ++half;
  const uint64_t mask = (1ull << half) - 1;
  uint64_t x = i;
  do {
    uint64_t l = x >> half, r = x & mask;
    for (int round = 0; round < 4; ++round) {
      const uint64_t f = mix64(r ^ key ^ (static_cast<uint64_t>(round) << 56)) & mask;
      const uint64_t nl = r;
      r = l ^ f;
      l = nl;
    }
    x = (l << half) | r;
  } while (x >= n);
  return x;
}

class TokenShards {
 public:
  TokenShards(const std::vector<std::string>& paths, int seq_len, int rank, int world, uint64_t seed, bool shuffle, int depth)
      : seq_(seq_len), rank_(rank), world_(world), seed_(seed), shuffle_(shuffle), depth_(depth < 0 ? 0 : depth) {
    if (seq_len <= 0) throw std::invalid_argument("TokenShards: seq_len must be positive");
    if (world <= 0 || rank < 0 || rank >= world) throw std::invalid_argument("TokenShards: bad rank / world");
    if (paths.empty()) throw std::invalid_argument("TokenShards: no shard given");
    try {
      for (const auto& p : paths) open_shard(p);
    } catch (...) {
      unmap_all();
      throw;
    }
    if (total_ == 0) {
      unmap_all();
      throw std::invalid_argument("TokenShards: no shard holds seq_len tokens");
    }
  }
  ~TokenShards() {
    stop_worker();
    unmap_all();
  }
  TokenShards(const TokenShards&) = delete;
  TokenShards& operator=(const TokenShards&) = delete;

  py::array_t<int32_t> next_rows(int rows, int seq_len) {
    if (seq_len != seq_) throw std::invalid_argument("TokenShards: seq_len differs from the one the windows were cut for");
    if (rows <= 0) throw std::invalid_argument("TokenShards: rows must be positive");
    py::array_t<int32_t> out({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(seq_)});
    int32_t* dst = out.mutable_data();
    {
      py::gil_scoped_release nogil;
      fetch(dst, rows);
    }
    return out;
  }

  // Fills caller memory (a pinned staging buffer, say): `rows * seq_len` int32 at `ptr`.
  void next_into(uintptr_t ptr, int rows) {
    if (rows <= 0 || ptr == 0) throw std::invalid_argument("TokenShards: bad destination");
    py::gil_scoped_release nogil;
    fetch(reinterpret_cast<int32_t*>(ptr), rows);
  }

  uint64_t cursor() const { return consumed_.load(); }
  uint64_t global_cursor() const { return consumed_.load() * static_cast<uint64_t>(world_); }
  void seek(uint64_t global) {
    std::lock_guard<std::mutex> one_consumer(consumer_mu_);
    stop_worker();
    ring_.clear();
    consumed_ = global / static_cast<uint64_t>(world_);
    produced_ = consumed_.load();
  }
  uint64_t windows() const { return total_; }
  uint64_t tokens() const {
    uint64_t n = 0;
    for (const auto& s : shards_) n += s.count;
    return n;
  }
  uint32_t vocab() const { return vocab_; }
  uint64_t window_of(uint64_t global_row) const { return locate(global_row); }
  uint64_t prefetched() const { return prefetched_.load(); }

 private:
  void open_shard(const std::string& path) {
    Shard s;
    s.path = path;
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) throw std::runtime_error("TokenShards: cannot open " + path);
    struct stat st {};
    if (::fstat(fd, &st) != 0 || st.st_size < 20) {
      ::close(fd);
      throw std::runtime_error("TokenShards: " + path + " is shorter than a shard header");
    }
    s.bytes = static_cast<size_t>(st.st_size);
    void* m = ::mmap(nullptr, s.bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) throw std::runtime_error("TokenShards: cannot map " + path);
    s.base = static_cast<const uint8_t*>(m);
    shards_.push_back(s);                 // from here on unmap_all() owns the mapping
    Shard& t = shards_.back();
    if (std::memcmp(t.base, "NXTK", 4) != 0) throw std::runtime_error("TokenShards: " + path + " is not an NXTK shard");
    uint32_t version = 0;
    std::memcpy(&version, t.base + 4, 4);
    std::memcpy(&t.vocab, t.base + 8, 4);
    std::memcpy(&t.count, t.base + 12, 8);
    if (version != 1) throw std::runtime_error("TokenShards: " + path + " has version " + std::to_string(version));
    t.width = t.vocab <= 65536 ? 2 : 4;
    if (t.count > (t.bytes - 20) / static_cast<size_t>(t.width)) throw std::runtime_error("TokenShards: " + path + " is truncated");
    t.data = t.base + 20;
    t.first_window = total_;
    t.windows = t.count / static_cast<uint64_t>(seq_);
    total_ += t.windows;
    if (t.vocab > vocab_) vocab_ = t.vocab;
    ::madvise(const_cast<uint8_t*>(t.base), t.bytes, MADV_WILLNEED);
  }
  void unmap_all() {
    for (auto& s : shards_)
      if (s.base != nullptr) ::munmap(const_cast<uint8_t*>(s.base), s.bytes);
    shards_.clear();
  }

  uint64_t locate(uint64_t global_row) const {
    const uint64_t epoch = global_row / total_, pos = global_row % total_;
    return shuffle_ ? permute(pos, total_, mix64(seed_ ^ mix64(epoch))) : pos;
  }

  void decode_row(uint64_t local_row, int32_t* dst) const {
    const uint64_t w = locate(local_row * static_cast<uint64_t>(world_) + static_cast<uint64_t>(rank_));
    size_t lo = 0, hi = shards_.size() - 1;   // last shard whose first window is <= w
    while (lo < hi) {
      const size_t mid = (lo + hi + 1) / 2;
      if (shards_[mid].first_window <= w) lo = mid; else hi = mid - 1;
    }
    const Shard& s = shards_[lo];
    const uint64_t off = (w - s.first_window) * static_cast<uint64_t>(seq_);
    if (s.width == 2) {
      const uint16_t* src = reinterpret_cast<const uint16_t*>(s.data) + off;
      for (int i = 0; i < seq_; ++i) dst[i] = static_cast<int32_t>(src[i]);
    } else {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(s.data) + off;
      for (int i = 0; i < seq_; ++i) dst[i] = static_cast<int32_t>(src[i]);
    }
  }

  struct Batch { uint64_t first = 0; int rows = 0; std::vector<int32_t> data; };

  void fetch(int32_t* dst, int rows) {
    std::lock_guard<std::mutex> one_consumer(consumer_mu_);   // calls from several threads are served one at a time
    if (depth_ > 0) {
      if (rows != worker_rows_) {          // first call, or the batch shape changed: restart the read-ahead
        stop_worker();
        ring_.clear();
        produced_ = consumed_.load();
        worker_rows_ = rows;
        start_worker();
      }
      std::unique_lock<std::mutex> lk(mu_);
      ready_.wait(lk, [&] { return !ring_.empty(); });
      Batch b = std::move(ring_.front());
      ring_.pop_front();
      lk.unlock();
      space_.notify_one();
      std::memcpy(dst, b.data.data(), b.data.size() * sizeof(int32_t));
      prefetched_.fetch_add(1);
    } else {
      const uint64_t first = consumed_.load();
      for (int r = 0; r < rows; ++r) decode_row(first + static_cast<uint64_t>(r), dst + static_cast<size_t>(r) * seq_);
    }
    consumed_.fetch_add(static_cast<uint64_t>(rows));
  }

  void start_worker() {
    stop_ = false;
    worker_ = std::thread([this] {
      while (true) {
        {
          std::unique_lock<std::mutex> lk(mu_);
          space_.wait(lk, [&] { return stop_ || static_cast<int>(ring_.size()) < depth_; });
          if (stop_) return;
        }
        Batch b;
        b.first = produced_;
        b.rows = worker_rows_;
        b.data.resize(static_cast<size_t>(worker_rows_) * seq_);
        for (int r = 0; r < worker_rows_; ++r)
          decode_row(b.first + static_cast<uint64_t>(r), b.data.data() + static_cast<size_t>(r) * seq_);
        produced_ += static_cast<uint64_t>(worker_rows_);
        {
          std::lock_guard<std::mutex> lk(mu_);
          ring_.push_back(std::move(b));
        }
        ready_.notify_one();
      }
    });
  }
  void stop_worker() {
    if (!worker_.joinable()) return;
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    space_.notify_all();
    worker_.join();
    worker_rows_ = -1;
  }

  int seq_, rank_, world_;
  uint64_t seed_;
  bool shuffle_;
  int depth_;
  std::vector<Shard> shards_;
  uint64_t total_ = 0;
  uint32_t vocab_ = 0;
  std::atomic<uint64_t> consumed_{0};      // rows handed out by this rank
  uint64_t produced_ = 0;                  // rows decoded by the worker (worker thread only, or while it is stopped)
  std::atomic<uint64_t> prefetched_{0};
  int worker_rows_ = -1;
  std::thread worker_;
  std::mutex mu_, consumer_mu_;
  std::condition_variable ready_, space_;
  std::deque<Batch> ring_;
  bool stop_ = false;
};

}  // namespace

void bind_token_data(py::module_& m) {
  py::class_<TokenShards>(m, "TokenShards")
      .def(py::init<const std::vector<std::string>&, int, int, int, uint64_t, bool, int>(), py::arg("paths"), py::arg("seq_len"),
           py::arg("rank") = 0, py::arg("world") = 1, py::arg("seed") = 0, py::arg("shuffle") = false, py::arg("depth") = 2)
      .def("next_rows", &TokenShards::next_rows)
      .def("next_into", &TokenShards::next_into)
      .def("cursor", &TokenShards::cursor)
      .def("global_cursor", &TokenShards::global_cursor)
      .def("seek", &TokenShards::seek)
      .def("windows", &TokenShards::windows)
      .def("tokens", &TokenShards::tokens)
      .def("vocab", &TokenShards::vocab)
      .def("window_of", &TokenShards::window_of)
      .def("prefetched", &TokenShards::prefetched);
  m.def("permute_index", &permute, "Keyed bijection on [0, n) (Feistel network with cycle walking)");
}
