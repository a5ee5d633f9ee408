// Host runtime pieces: caching allocator (64-byte aligned, power-of-two size classes, statistics),
// static memory planner (greedy-by-size best-fit arena from tensor lifetimes), profiler
// (interval records, per-name totals, op counters, Chrome trace export) and the memory ledger
// (current / peak bytes per label and memory space).
// Parity: include/nexus/core/allocator.hpp:36-99, include/nexus/memory/planner.hpp:18-54,
// include/nexus/prof/{timer,counters,trace,memory_ledger}.hpp + src/prof/prof.cpp of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <thread>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

// ------------------------------------------------------------------------------------ allocator
class CachingAllocator {
 public:
  static constexpr size_t kAlign = 64;
  ~CachingAllocator() { release_cached(); }

  uintptr_t allocate(size_t bytes) {
    const size_t cls = size_class(bytes);
    std::lock_guard<std::mutex> lk(mu_);
    ++requests_;
    auto& fl = free_[cls];
    void* p;
    if (!fl.empty()) {
      p = fl.back();
      fl.pop_back();
      ++hits_;
      cached_bytes_ -= cls;
    } else {
      p = std::aligned_alloc(kAlign, cls);
      if (p == nullptr) throw std::bad_alloc();
      ++system_allocs_;
      reserved_bytes_ += cls;
    }
    live_[p] = {cls, bytes};
    in_use_bytes_ += cls;
    requested_bytes_ += bytes;
    peak_in_use_ = std::max(peak_in_use_, in_use_bytes_);
    return reinterpret_cast<uintptr_t>(p);
  }
  void deallocate(uintptr_t addr) {
    void* p = reinterpret_cast<void*>(addr);
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) throw std::invalid_argument("deallocate: unknown pointer");
    free_[it->second.first].push_back(p);
    in_use_bytes_ -= it->second.first;
    requested_bytes_ -= it->second.second;
    cached_bytes_ += it->second.first;
    live_.erase(it);
  }
  void release_cached() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : free_) {
      for (void* p : kv.second) {
        std::free(p);
        reserved_bytes_ -= kv.first;
      }
      kv.second.clear();
    }
    cached_bytes_ = 0;
  }
  py::dict stats() {
    std::lock_guard<std::mutex> lk(mu_);
    py::dict d;
    d["requests"] = requests_;
    d["hits"] = hits_;
    d["system_allocs"] = system_allocs_;
    d["in_use_bytes"] = in_use_bytes_;
    d["cached_bytes"] = cached_bytes_;
    d["reserved_bytes"] = reserved_bytes_;
    d["peak_in_use_bytes"] = peak_in_use_;
    // internal fragmentation: share of in-use bytes that is rounding slack
    d["fragmentation"] = in_use_bytes_ ? 1.0 - static_cast<double>(requested_bytes_) / in_use_bytes_ : 0.0;
    return d;
  }
  static size_t size_class(size_t bytes) {
    size_t c = kAlign;
    while (c < bytes) c <<= 1;
    return c;
  }

 private:
  std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
  std::unordered_map<void*, std::pair<size_t, size_t>> live_;
  size_t requests_ = 0, hits_ = 0, system_allocs_ = 0, in_use_bytes_ = 0, cached_bytes_ = 0, reserved_bytes_ = 0,
         peak_in_use_ = 0, requested_bytes_ = 0;
};

// -------------------------------------------------------------------------------------- planner
struct Lifetime {
  int64_t bytes, first, last;
};

// Greedy by size: place the largest tensor first at the lowest offset that does not overlap (in
// time and space) anything already placed.  Returns (offsets, arena_bytes).
std::pair<std::vector<int64_t>, int64_t> plan_memory(const std::vector<std::tuple<int64_t, int64_t, int64_t>>& lt,
                                                     int64_t alignment) {
  const size_t n = lt.size();
  std::vector<size_t> order(n);
  for (size_t i = 0; i < n; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(),
                   [&](size_t a, size_t b) { return std::get<0>(lt[a]) > std::get<0>(lt[b]); });
  std::vector<int64_t> offset(n, -1);
  int64_t arena = 0;
  auto up = [&](int64_t v) { return (v + alignment - 1) / alignment * alignment; };
  for (size_t idx : order) {
    const int64_t bytes = up(std::max<int64_t>(std::get<0>(lt[idx]), 1));
    const int64_t f = std::get<1>(lt[idx]), l = std::get<2>(lt[idx]);
    std::vector<std::pair<int64_t, int64_t>> busy;  // occupied [begin, end) among time-overlapping tensors
    for (size_t j = 0; j < n; ++j) {
      if (offset[j] < 0) continue;
      if (std::get<2>(lt[j]) < f || std::get<1>(lt[j]) > l) continue;
      busy.emplace_back(offset[j], offset[j] + up(std::max<int64_t>(std::get<0>(lt[j]), 1)));
    }
    std::sort(busy.begin(), busy.end());
    int64_t best = -1, best_gap = -1, cursor = 0;
    for (const auto& b : busy) {
      if (b.first - cursor >= bytes) {
        const int64_t gap = b.first - cursor;
        if (best < 0 || gap < best_gap) {
          best = cursor;
          best_gap = gap;
        }
      }
      cursor = std::max(cursor, b.second);
    }
    if (best < 0) best = cursor;
    offset[idx] = best;
    arena = std::max(arena, best + bytes);
  }
  return {offset, arena};
}

// ------------------------------------------------------------------------------------- profiler
struct Interval {
  std::string name, category;
  uint64_t thread;
  int64_t start_ns, duration_ns;
};

class Profiler {
 public:
  void enable(bool on) { enabled_ = on; }
  bool enabled() const { return enabled_; }
  static int64_t now_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
        .count();
  }
  void record(const std::string& name, const std::string& cat, int64_t start_ns, int64_t dur_ns) {
    if (!enabled_) return;
    const uint64_t tid = std::hash<std::thread::id>{}(std::this_thread::get_id()) & 0xffff;
    std::lock_guard<std::mutex> lk(mu_);
    records_.push_back({name, cat, tid, start_ns, dur_ns});
    auto& t = totals_[name];
    t.calls += 1;
    t.total += dur_ns;
    t.min = t.calls == 1 ? dur_ns : std::min(t.min, dur_ns);
    t.max = std::max(t.max, dur_ns);
  }
  void count(const std::string& op, double flops, double bytes) {
    std::lock_guard<std::mutex> lk(mu_);
    auto& c = counters_[op];
    c.calls += 1;
    c.flops += flops;
    c.bytes += bytes;
  }
  py::dict totals() {
    std::lock_guard<std::mutex> lk(mu_);
    py::dict d;
    for (auto& kv : totals_) {
      py::dict e;
      e["calls"] = kv.second.calls;
      e["total_ns"] = kv.second.total;
      e["min_ns"] = kv.second.min;
      e["max_ns"] = kv.second.max;
      d[py::str(kv.first)] = e;
    }
    return d;
  }
  py::dict counters() {
    std::lock_guard<std::mutex> lk(mu_);
    py::dict d;
    for (auto& kv : counters_) {
      py::dict e;
      e["calls"] = kv.second.calls;
      e["flops"] = kv.second.flops;
      e["bytes"] = kv.second.bytes;
      d[py::str(kv.first)] = e;
    }
    return d;
  }
  size_t dump_chrome_trace(const std::string& path) {
    std::lock_guard<std::mutex> lk(mu_);
    std::ofstream out(path);
    if (!out) throw std::runtime_error("cannot open " + path);
    out << "{\"traceEvents\":[";
    bool first = true;
    for (const auto& r : records_) {
      if (!first) out << ",";
      first = false;
      out << "{\"name\":\"" << escape(r.name) << "\",\"cat\":\"" << escape(r.category) << "\",\"ph\":\"X\",\"ts\":"
          << r.start_ns / 1000.0 << ",\"dur\":" << r.duration_ns / 1000.0 << ",\"pid\":0,\"tid\":" << r.thread << "}";
    }
    out << "]}";
    return records_.size();
  }
  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    records_.clear();
    totals_.clear();
    counters_.clear();
  }

 private:
  static std::string escape(const std::string& s) {
    std::string o;
    for (char c : s) {
      if (c == '"' || c == '\\') o.push_back('\\');
      o.push_back(c);
    }
    return o;
  }
  struct Total {
    int64_t calls = 0, total = 0, min = 0, max = 0;
  };
  struct Counter {
    int64_t calls = 0;
    double flops = 0, bytes = 0;
  };
  bool enabled_ = false;
  std::mutex mu_;
  std::vector<Interval> records_;
  std::map<std::string, Total> totals_;
  std::map<std::string, Counter> counters_;
};

Profiler& profiler() {
  static Profiler p;
  return p;
}

// --------------------------------------------------------------------------------------- ledger
// labels: Parameter, Gradient, OptimizerState, Activation, Temporary, CommBuffer, KvCache
// spaces: Host, PinnedHost, Device
class MemoryLedger {
 public:
  void add(int label, int space, int64_t bytes) {
    check(label, space);
    std::lock_guard<std::mutex> lk(mu_);
    cur_[label][space] += bytes;
    peak_[label][space] = std::max(peak_[label][space], cur_[label][space]);
  }
  int64_t current(int label, int space) {
    check(label, space);
    std::lock_guard<std::mutex> lk(mu_);
    return cur_[label][space];
  }
  int64_t peak(int label, int space) {
    check(label, space);
    std::lock_guard<std::mutex> lk(mu_);
    return peak_[label][space];
  }
  void reset() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& r : cur_) for (auto& v : r) v = 0;
    for (auto& r : peak_) for (auto& v : r) v = 0;
  }

 private:
  static void check(int label, int space) {
    if (label < 0 || label >= 7 || space < 0 || space >= 3) throw std::out_of_range("memory ledger index");
  }
  std::mutex mu_;
  int64_t cur_[7][3] = {};
  int64_t peak_[7][3] = {};
};

MemoryLedger& ledger() {
  static MemoryLedger l;
  return l;
}

}  // namespace

void bind_runtime(py::module_& m) {
  py::class_<CachingAllocator>(m, "HostCachingAllocator")
      .def(py::init<>())
      .def("allocate", &CachingAllocator::allocate)
      .def("deallocate", &CachingAllocator::deallocate)
      .def("release_cached", &CachingAllocator::release_cached)
      .def("stats", &CachingAllocator::stats)
      .def_static("size_class", &CachingAllocator::size_class);
  m.def("plan_memory", &plan_memory, py::arg("lifetimes"), py::arg("alignment") = 256,
        "lifetimes: [(bytes, first_use, last_use)] -> (offsets, arena_bytes)");
  m.def("prof_enable", [](bool on) { profiler().enable(on); });
  m.def("prof_enabled", [] { return profiler().enabled(); });
  m.def("prof_now_ns", [] { return Profiler::now_ns(); });
  m.def("prof_record", [](const std::string& n, const std::string& c, int64_t s, int64_t d) { profiler().record(n, c, s, d); });
  m.def("prof_count", [](const std::string& op, double f, double b) { profiler().count(op, f, b); });
  m.def("prof_totals", [] { return profiler().totals(); });
  m.def("prof_counters", [] { return profiler().counters(); });
  m.def("prof_dump_chrome_trace", [](const std::string& p) { return profiler().dump_chrome_trace(p); });
  m.def("prof_clear", [] { profiler().clear(); });
  m.def("ledger_add", [](int l, int s, int64_t b) { ledger().add(l, s, b); });
  m.def("ledger_current", [](int l, int s) { return ledger().current(l, s); });
  m.def("ledger_peak", [](int l, int s) { return ledger().peak(l, s); });
  m.def("ledger_reset", [] { ledger().reset(); });
}
