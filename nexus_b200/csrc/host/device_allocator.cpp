// Stream-aware caching allocator for device memory, and the CPU feature / thread-pool / quantised GEMV
// runtime.
//
// Allocator design (no virtual-memory expandable segments): requests are rounded to 512 bytes; requests of
// at most 1 MiB come from 2 MiB segments of the small pool, larger ones from segments of at least 20 MiB
// (or the rounded request) of the large pool.  A free block is split when the remainder is worth keeping
// and merged with free neighbours of the same segment when it returns.  Free lists are per stream: a block
// is reused only on the stream it was allocated for, unless `record_stream` noted other users, in which
// case it returns to the pool only after the events recorded on those streams have completed.  On
// out-of-memory the cache is emptied and the request retried once.  The backing store is either the host
// heap (tests, pinned pools) or the CUDA runtime looked up in the running process.
// Parity: include/nexus/cuda/caching_allocator.hpp:5-60, src/cuda/caching_allocator.cpp of the reference.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <condition_variable>
#include <functional>
#include <fstream>
#include <vector>

#include <dlfcn.h>
#if defined(__x86_64__)
#include <cpuid.h>
#include <immintrin.h>
#endif

namespace py = pybind11;

namespace {

constexpr size_t kRound = 512, kSmallLimit = 1 << 20, kSmallSegment = 2 << 20, kLargeSegment = 20 << 20;

struct Backing {
  virtual ~Backing() = default;
  virtual void* alloc(size_t bytes) = 0;  // nullptr on failure
  virtual void release(void* p) = 0;
  virtual uint64_t record(uint64_t stream) = 0;  // returns an event id (0: none needed)
  virtual bool done(uint64_t event) = 0;
};

struct HostBacking final : Backing {
  size_t limit, used = 0;
  std::map<void*, size_t> sizes;
  explicit HostBacking(size_t limit_bytes) : limit(limit_bytes) {}
  void* alloc(size_t bytes) override {
    if (limit && used + bytes > limit) return nullptr;
    void* p = std::aligned_alloc(kRound, bytes);
    if (p) {
      used += bytes;
      sizes[p] = bytes;
    }
    return p;
  }
  void release(void* p) override {
    used -= sizes[p];
    sizes.erase(p);
    std::free(p);
  }
  uint64_t record(uint64_t) override { return 0; }
  bool done(uint64_t) override { return true; }
};

// CUDA runtime entry points resolved from the process image (torch has loaded libcudart already).
struct CudaBacking final : Backing {
  using MallocFn = int (*)(void**, size_t);
  using FreeFn = int (*)(void*);
  using EvCreateFn = int (*)(void**, unsigned);
  using EvRecordFn = int (*)(void*, void*);
  using EvQueryFn = int (*)(void*);
  using EvDestroyFn = int (*)(void*);
  MallocFn malloc_ = nullptr;
  FreeFn free_ = nullptr;
  EvCreateFn ev_create_ = nullptr;
  EvRecordFn ev_record_ = nullptr;
  EvQueryFn ev_query_ = nullptr;
  EvDestroyFn ev_destroy_ = nullptr;
  std::map<uint64_t, void*> events;
  uint64_t next_event = 1;
  CudaBacking() {
    auto sym = [](const char* name) -> void* {
      void* s = dlsym(RTLD_DEFAULT, name);
      if (!s) {
        void* lib = dlopen("libcudart.so.12", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libcudart.so", RTLD_NOW | RTLD_GLOBAL);
        if (lib) s = dlsym(lib, name);
      }
      if (!s) throw std::runtime_error(std::string("CUDA runtime symbol not found: ") + name);
      return s;
    };
    malloc_ = reinterpret_cast<MallocFn>(sym("cudaMalloc"));
    free_ = reinterpret_cast<FreeFn>(sym("cudaFree"));
    ev_create_ = reinterpret_cast<EvCreateFn>(sym("cudaEventCreateWithFlags"));
    ev_record_ = reinterpret_cast<EvRecordFn>(sym("cudaEventRecord"));
    ev_query_ = reinterpret_cast<EvQueryFn>(sym("cudaEventQuery"));
    ev_destroy_ = reinterpret_cast<EvDestroyFn>(sym("cudaEventDestroy"));
  }
  void* alloc(size_t bytes) override {
    void* p = nullptr;
    return malloc_(&p, bytes) == 0 ? p : nullptr;
  }
  void release(void* p) override { free_(p); }
  uint64_t record(uint64_t stream) override {
    void* ev = nullptr;
    if (ev_create_(&ev, 2 /* cudaEventDisableTiming */) != 0) return 0;
    ev_record_(ev, reinterpret_cast<void*>(stream));
    events[next_event] = ev;
    return next_event++;
  }
  bool done(uint64_t event) override {
    auto it = events.find(event);
    if (it == events.end()) return true;
    if (ev_query_(it->second) != 0) return false;  // cudaErrorNotReady
    ev_destroy_(it->second);
    events.erase(it);
    return true;
  }
};

struct Block {
  uint8_t* ptr;
  size_t size;
  uint64_t stream;
  bool small, free_ = true;
  Block *prev = nullptr, *next = nullptr;  // neighbours inside the segment
  std::set<uint64_t> users;                // other streams that touched the block
};

struct Stats {
  uint64_t allocations = 0, cache_hits = 0, segments = 0, splits = 0, merges = 0, oom_retries = 0;
  uint64_t allocated_bytes = 0, reserved_bytes = 0, peak_allocated = 0, peak_reserved = 0, deferred = 0;
};

class DeviceCachingAllocator {
 public:
  DeviceCachingAllocator(const std::string& backing, size_t limit) {
    if (backing == "host") backing_ = std::make_unique<HostBacking>(limit);
    else if (backing == "cuda") backing_ = std::make_unique<CudaBacking>();
    else throw std::invalid_argument("backing must be 'host' or 'cuda'");
  }
  ~DeviceCachingAllocator() {
    for (auto& kv : segments_) backing_->release(kv.first);
  }

  uint64_t alloc(size_t bytes, uint64_t stream) {
    std::lock_guard<std::mutex> g(mu_);
    process_deferred();
    const size_t size = std::max(kRound, (bytes + kRound - 1) / kRound * kRound);
    const bool small = size <= kSmallLimit;
    Block* b = take_free(size, stream, small);
    if (b) ++stats_.cache_hits;
    if (!b) b = new_segment(size, stream, small);
    if (!b) {  // out of memory: drop every cached segment and try once more
      ++stats_.oom_retries;
      empty_cache_locked();
      b = new_segment(size, stream, small);
      if (!b) throw std::runtime_error("out of device memory: " + std::to_string(bytes) + " bytes requested");
    }
    const size_t rest = b->size - size;
    if (rest >= (small ? kRound : kSmallLimit + kRound)) {
      Block* r = new Block{b->ptr + size, rest, b->stream, b->small};
      r->prev = b;
      r->next = b->next;
      if (b->next) b->next->prev = r;
      b->next = r;
      b->size = size;
      free_[key(r)].insert(r);
      ++stats_.splits;
    }
    b->free_ = false;
    live_[b->ptr] = b;
    ++stats_.allocations;
    stats_.allocated_bytes += b->size;
    stats_.peak_allocated = std::max(stats_.peak_allocated, stats_.allocated_bytes);
    return reinterpret_cast<uint64_t>(b->ptr);
  }

  void free(uint64_t p) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(reinterpret_cast<uint8_t*>(p));
    if (it == live_.end()) throw std::invalid_argument("free of a pointer this allocator does not own");
    Block* b = it->second;
    live_.erase(it);
    stats_.allocated_bytes -= b->size;
    if (!b->users.empty()) {  // other streams may still be reading: wait for their events
      std::vector<uint64_t> evs;
      for (uint64_t s : b->users) {
        const uint64_t e = backing_->record(s);
        if (e) evs.push_back(e);
      }
      b->users.clear();
      if (!evs.empty()) {
        deferred_.push_back({b, evs});
        ++stats_.deferred;
        return;
      }
    }
    release_block(b);
  }

  void record_stream(uint64_t p, uint64_t stream) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(reinterpret_cast<uint8_t*>(p));
    if (it == live_.end()) throw std::invalid_argument("record_stream of an unknown pointer");
    if (stream != it->second->stream) it->second->users.insert(stream);
  }

  void empty_cache() {
    std::lock_guard<std::mutex> g(mu_);
    process_deferred();
    empty_cache_locked();
  }

  py::dict stats() {
    std::lock_guard<std::mutex> g(mu_);
    py::dict d;
    d["allocations"] = stats_.allocations;
    d["cache_hits"] = stats_.cache_hits;
    d["segments"] = stats_.segments;
    d["splits"] = stats_.splits;
    d["merges"] = stats_.merges;
    d["oom_retries"] = stats_.oom_retries;
    d["allocated_bytes"] = stats_.allocated_bytes;
    d["reserved_bytes"] = stats_.reserved_bytes;
    d["peak_allocated_bytes"] = stats_.peak_allocated;
    d["peak_reserved_bytes"] = stats_.peak_reserved;
    d["deferred_frees"] = stats_.deferred;
    d["pending_frees"] = static_cast<uint64_t>(deferred_.size());
    d["live_blocks"] = static_cast<uint64_t>(live_.size());
    size_t cached = 0, largest = 0;
    for (auto& kv : free_)
      for (Block* b : kv.second) {
        cached += b->size;
        largest = std::max(largest, b->size);
      }
    d["cached_bytes"] = static_cast<uint64_t>(cached);
    d["fragmentation"] = cached ? 1.0 - static_cast<double>(largest) / static_cast<double>(cached) : 0.0;
    return d;
  }

 private:
  struct BySize {
    bool operator()(const Block* a, const Block* b) const {
      return a->size != b->size ? a->size < b->size : a->ptr < b->ptr;
    }
  };
  using FreeSet = std::set<Block*, BySize>;
  struct Deferred {
    Block* block;
    std::vector<uint64_t> events;
  };

  static std::pair<uint64_t, bool> key(const Block* b) { return {b->stream, b->small}; }

  Block* take_free(size_t size, uint64_t stream, bool small) {
    auto it = free_.find({stream, small});
    if (it == free_.end()) return nullptr;
    Block probe{nullptr, size, stream, small};
    auto f = it->second.lower_bound(&probe);
    if (f == it->second.end()) return nullptr;
    Block* b = *f;
    if (!small && b->size > 2 * size && b->size - size > kLargeSegment) return nullptr;  // do not waste a huge block
    it->second.erase(f);
    return b;
  }

  Block* new_segment(size_t size, uint64_t stream, bool small) {
    const size_t seg = small ? kSmallSegment : std::max(kLargeSegment, size);
    void* p = backing_->alloc(seg);
    if (!p && !small && seg > size) p = backing_->alloc(size);  // no room for slack: exact size
    if (!p) return nullptr;
    const size_t got = (seg > size && !small && segments_.count(p) == 0) ? seg : seg;
    segments_[p] = got;
    ++stats_.segments;
    stats_.reserved_bytes += got;
    stats_.peak_reserved = std::max(stats_.peak_reserved, stats_.reserved_bytes);
    return new Block{static_cast<uint8_t*>(p), got, stream, small};
  }

  void release_block(Block* b) {
    b->free_ = true;
    for (Block* n : {b->prev, b->next}) {
      if (n && n->free_) {
        free_[key(n)].erase(n);
        if (n == b->prev) {
          n->size += b->size;
          n->next = b->next;
          if (b->next) b->next->prev = n;
          delete b;
          b = n;
        } else {
          b->size += n->size;
          b->next = n->next;
          if (n->next) n->next->prev = b;
          delete n;
        }
        ++stats_.merges;
      }
    }
    free_[key(b)].insert(b);
  }

  void process_deferred() {
    for (size_t i = 0; i < deferred_.size();) {
      auto& d = deferred_[i];
      d.events.erase(std::remove_if(d.events.begin(), d.events.end(), [&](uint64_t e) { return backing_->done(e); }),
                     d.events.end());
      if (d.events.empty()) {
        release_block(d.block);
        deferred_.erase(deferred_.begin() + static_cast<long>(i));
      } else {
        ++i;
      }
    }
  }

  void empty_cache_locked() {
    for (auto& kv : free_) {
      for (auto it = kv.second.begin(); it != kv.second.end();) {
        Block* b = *it;
        if (b->prev == nullptr && b->next == nullptr) {  // the whole segment is free
          stats_.reserved_bytes -= segments_[b->ptr];
          segments_.erase(b->ptr);
          backing_->release(b->ptr);
          delete b;
          it = kv.second.erase(it);
        } else {
          ++it;
        }
      }
    }
  }

  std::unique_ptr<Backing> backing_;
  std::mutex mu_;
  std::map<std::pair<uint64_t, bool>, FreeSet> free_;
  std::map<uint8_t*, Block*> live_;
  std::map<void*, size_t> segments_;
  std::vector<Deferred> deferred_;
  Stats stats_;
};

// =================================================================================================
// CPU features and topology
// =================================================================================================
py::dict cpu_features() {
  py::dict d;
  bool sse42 = false, avx = false, avx2 = false, fma = false, f16c = false, avx512f = false, avx512bw = false,
       avx512vnni = false, avx_vnni = false, amx_bf16 = false, bmi2 = false, os_avx = false;
  std::string vendor = "unknown", brand;
#if defined(__x86_64__)
  unsigned a, b, c, dd;
  if (__get_cpuid(0, &a, &b, &c, &dd)) {
    char v[13] = {0};
    std::memcpy(v, &b, 4);
    std::memcpy(v + 4, &dd, 4);
    std::memcpy(v + 8, &c, 4);
    vendor = v;
  }
  if (__get_cpuid(1, &a, &b, &c, &dd)) {
    sse42 = c & (1u << 20);
    fma = c & (1u << 12);
    f16c = c & (1u << 29);
    const bool osxsave = c & (1u << 27);
    if (osxsave) {
      unsigned lo, hi;
      __asm__ volatile("xgetbv" : "=a"(lo), "=d"(hi) : "c"(0));
      os_avx = (lo & 6u) == 6u;
    }
    avx = (c & (1u << 28)) && os_avx;
  }
  if (__get_cpuid_count(7, 0, &a, &b, &c, &dd)) {
    avx2 = (b & (1u << 5)) && os_avx;
    bmi2 = b & (1u << 8);
    avx512f = (b & (1u << 16)) && os_avx;
    avx512bw = (b & (1u << 30)) && os_avx;
    avx512vnni = (c & (1u << 11)) && os_avx;
    amx_bf16 = dd & (1u << 22);
  }
  if (__get_cpuid_count(7, 1, &a, &b, &c, &dd)) avx_vnni = a & (1u << 4);
  char br[49] = {0};
  for (unsigned i = 0; i < 3; ++i) {
    unsigned r[4];
    if (__get_cpuid(0x80000002u + i, &r[0], &r[1], &r[2], &r[3])) std::memcpy(br + 16 * i, r, 16);
  }
  brand = br;
#endif
  d["vendor"] = vendor;
  d["brand"] = brand;
  d["sse42"] = sse42;
  d["avx"] = avx;
  d["avx2"] = avx2;
  d["fma"] = fma;
  d["f16c"] = f16c;
  d["bmi2"] = bmi2;
  d["avx512f"] = avx512f;
  d["avx512bw"] = avx512bw;
  d["avx512vnni"] = avx512vnni;
  d["avx_vnni"] = avx_vnni;
  d["amx_bf16"] = amx_bf16;
  const unsigned logical = std::max(1u, std::thread::hardware_concurrency());
  d["logical_cores"] = logical;
  // physical cores and caches from sysfs (fall back to the logical count)
  std::set<std::pair<int, int>> cores;
  std::set<int> nodes;
  for (unsigned cpu = 0; cpu < logical; ++cpu) {
    const std::string base = "/sys/devices/system/cpu/cpu" + std::to_string(cpu) + "/topology/";
    std::ifstream fc(base + "core_id"), fp(base + "physical_package_id");
    int core = -1, pkg = 0;
    if (fc >> core) {
      fp >> pkg;
      cores.insert({pkg, core});
    }
  }
  for (int n = 0; n < 64; ++n) {
    std::ifstream f("/sys/devices/system/node/node" + std::to_string(n) + "/cpulist");
    if (f.good()) nodes.insert(n);
  }
  d["physical_cores"] = cores.empty() ? logical : static_cast<unsigned>(cores.size());
  d["smt"] = !cores.empty() && cores.size() < logical;
  d["numa_nodes"] = nodes.empty() ? 1 : static_cast<int>(nodes.size());
  auto cache = [](int index) -> long {
    std::ifstream f("/sys/devices/system/cpu/cpu0/cache/index" + std::to_string(index) + "/size");
    std::string s;
    if (!(f >> s) || s.empty()) return 0;
    long v = std::atol(s.c_str());
    if (s.back() == 'K') v *= 1024;
    if (s.back() == 'M') v *= 1024 * 1024;
    return v;
  };
  d["l1d_bytes"] = cache(0);
  d["l2_bytes"] = cache(2);
  d["l3_bytes"] = cache(3);
  return d;
}

// =================================================================================================
// persistent thread pool with a static, deterministic partition
// =================================================================================================
class ThreadPool {
 public:
  explicit ThreadPool(int workers) : n_(std::max(1, workers)) {
    for (int w = 1; w < n_; ++w) threads_.emplace_back([this, w] { loop(w); });
  }
  ~ThreadPool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
      ++epoch_;
    }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  int size() const { return n_; }
  // fn(worker, begin, end) over [0, n) split into equal contiguous ranges (worker w gets range w)
  void run(int64_t n, const std::function<void(int, int64_t, int64_t)>& fn) {
    {
      std::lock_guard<std::mutex> g(mu_);
      fn_ = &fn;
      total_ = n;
      pending_ = n_ - 1;
      ++epoch_;
    }
    cv_.notify_all();
    part(0);
    std::unique_lock<std::mutex> g(mu_);
    done_.wait(g, [this] { return pending_ == 0; });
    fn_ = nullptr;
  }

 private:
  void part(int w) {
    const int64_t per = (total_ + n_ - 1) / n_;
    const int64_t b = std::min<int64_t>(total_, w * per), e = std::min<int64_t>(total_, b + per);
    if (b < e) (*fn_)(w, b, e);
  }
  void loop(int w) {
    uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [&] { return epoch_ != seen; });
        seen = epoch_;
        if (stop_) return;
      }
      part(w);
      {
        std::lock_guard<std::mutex> g(mu_);
        --pending_;
      }
      done_.notify_one();
    }
  }
  int n_;
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_, done_;
  const std::function<void(int, int64_t, int64_t)>* fn_ = nullptr;
  int64_t total_ = 0;
  int pending_ = 0;
  uint64_t epoch_ = 0;
  bool stop_ = false;
};

// y[m][n] = sum_k x[m][k] * w[n][k] (+ bias[n]); output columns are split over the workers, every dot
// product is accumulated in index order by one thread: the result does not depend on the thread count.
using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;

py::array_t<float> cpu_gemm_nt(ThreadPool& pool, FArr x, FArr w, py::object bias) {
  if (x.ndim() != 2 || w.ndim() != 2 || x.shape(1) != w.shape(1)) throw std::invalid_argument("gemm_nt: shapes");
  const int64_t M = x.shape(0), K = x.shape(1), N = w.shape(0);
  py::array_t<float> y({M, N});
  const float *xp = x.data(), *wp = w.data();
  const float* bp = nullptr;
  FArr b;
  if (!bias.is_none()) {
    b = bias.cast<FArr>();
    bp = b.data();
  }
  float* yp = y.mutable_data();
  {
    py::gil_scoped_release rel;
    pool.run(N, [&](int, int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n)
        for (int64_t m = 0; m < M; ++m) {
          const float* xr = xp + m * K;
          const float* wr = wp + n * K;
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          int64_t k = 0;
          for (; k + 8 <= K; k += 8)
            for (int j = 0; j < 8; ++j) acc[j] += xr[k + j] * wr[k + j];
          float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
          for (; k < K; ++k) s += xr[k] * wr[k];
          yp[m * N + n] = s + (bp ? bp[n] : 0.0f);
        }
    });
  }
  return y;
}

// The same product with the weights held as BF16 bit patterns (uint16, upper half of the FP32 word): half the
// weight bytes of cpu_gemm_nt, FP32 accumulation in the same index order.
py::array_t<float> cpu_gemm_nt_bf16(ThreadPool& pool, FArr x,
                                    py::array_t<uint16_t, py::array::c_style | py::array::forcecast> w, py::object bias) {
  if (x.ndim() != 2 || w.ndim() != 2 || x.shape(1) != w.shape(1)) throw std::invalid_argument("gemm_nt_bf16: shapes");
  const int64_t M = x.shape(0), K = x.shape(1), N = w.shape(0);
  py::array_t<float> y({M, N});
  const float* xp = x.data();
  const uint16_t* wp = w.data();
  const float* bp = nullptr;
  FArr b;
  if (!bias.is_none()) {
    b = bias.cast<FArr>();
    bp = b.data();
  }
  float* yp = y.mutable_data();
  {
    py::gil_scoped_release rel;
    pool.run(N, [&](int, int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n)
        for (int64_t m = 0; m < M; ++m) {
          const float* xr = xp + m * K;
          const uint16_t* wr = wp + n * K;
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          int64_t k = 0;
          for (; k + 8 <= K; k += 8)
            for (int j = 0; j < 8; ++j) {
              const uint32_t bits = static_cast<uint32_t>(wr[k + j]) << 16;
              float wv;
              std::memcpy(&wv, &bits, 4);
              acc[j] += xr[k + j] * wv;
            }
          float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
          for (; k < K; ++k) {
            const uint32_t bits = static_cast<uint32_t>(wr[k]) << 16;
            float wv;
            std::memcpy(&wv, &bits, 4);
            s += xr[k] * wv;
          }
          yp[m * N + n] = s + (bp ? bp[n] : 0.0f);
        }
    });
  }
  return y;
}

// Blocked ("flash") attention on the CPU, FP32: q [B, Tq, H, D], k / v [B, Tk, Hkv, D] (GQA: H a multiple of Hkv).
// One (batch, head, 64-row query block) per work item; key blocks of 64 with the online-softmax recurrence, so the
// [Tq, Tk] score matrix never exists.  Causal masking aligns the last query with the last key (Tq <= Tk), `window`
// > 0 limits each query to its last `window` keys, `softcap` > 0 passes scores through softcap * tanh(s / softcap),
// `alibi` (H slopes, may be empty) adds slope * (key - query position).  Returns (o [B, Tq, H, D], lse [B, H, Tq]).
py::tuple cpu_flash_attention(ThreadPool& pool, FArr q, FArr k, FArr v, bool causal, int window, double scale,
                              double softcap, FArr alibi) {
  if (q.ndim() != 4 || k.ndim() != 4 || v.ndim() != 4) throw std::invalid_argument("flash_attention: [B, T, H, D] tensors");
  const int64_t B = q.shape(0), Tq = q.shape(1), H = q.shape(2), D = q.shape(3);
  const int64_t Tk = k.shape(1), Hkv = k.shape(2);
  if (k.shape(0) != B || v.shape(0) != B || k.shape(3) != D || v.shape(3) != D || v.shape(1) != Tk || v.shape(2) != Hkv ||
      Hkv < 1 || H % Hkv)
    throw std::invalid_argument("flash_attention: shapes");
  if (alibi.size() != 0 && alibi.size() != H) throw std::invalid_argument("flash_attention: alibi needs one slope per head");
  py::array_t<float> o({B, Tq, H, D});
  py::array_t<float> lse({B, H, Tq});
  const float *qp = q.data(), *kp = k.data(), *vp = v.data();
  const float* ap = alibi.size() ? alibi.data() : nullptr;
  float* op = o.mutable_data();
  float* lp = lse.mutable_data();
  constexpr int64_t BQ = 64, BK = 64;
  const int64_t nqb = (Tq + BQ - 1) / BQ;
  const int64_t items = B * H * nqb;
  const int64_t shift = Tk - Tq;  // query i sits at key position i + shift
  {
    py::gil_scoped_release rel;
    pool.run(items, [&](int, int64_t i0, int64_t i1) {
      std::vector<float> s(BQ * BK), acc(BQ * D), mrow(BQ), lrow(BQ);
      for (int64_t it = i0; it < i1; ++it) {
        const int64_t qb = it % nqb, h = (it / nqb) % H, b = it / (nqb * H);
        const int64_t hk = h / (H / Hkv);
        const int64_t q0 = qb * BQ, rows = std::min(BQ, Tq - q0);
        std::fill(acc.begin(), acc.end(), 0.0f);
        std::fill(mrow.begin(), mrow.end(), -INFINITY);
        std::fill(lrow.begin(), lrow.end(), 0.0f);
        int64_t k_hi = Tk;
        if (causal) k_hi = std::min(Tk, q0 + rows + shift);
        int64_t k_lo = 0;
        if (window > 0) k_lo = std::max<int64_t>(0, q0 + shift - window + 1);
        for (int64_t k0 = (k_lo / BK) * BK; k0 < k_hi; k0 += BK) {
          const int64_t cols = std::min(BK, Tk - k0);
          for (int64_t r = 0; r < rows; ++r) {
            const float* qr = qp + ((b * Tq + q0 + r) * H + h) * D;
            const int64_t qpos = q0 + r + shift;
            for (int64_t c = 0; c < cols; ++c) {
              const int64_t kpos = k0 + c;
              float val = -INFINITY;
              const bool masked = (causal && kpos > qpos) || (window > 0 && kpos < qpos - window + 1);
              if (!masked) {
                const float* kr = kp + ((b * Tk + kpos) * Hkv + hk) * D;
                float d0 = 0.0f;
                for (int64_t e = 0; e < D; ++e) d0 += qr[e] * kr[e];
                val = d0 * static_cast<float>(scale);
                if (softcap > 0.0) val = static_cast<float>(softcap) * std::tanh(val / static_cast<float>(softcap));
                if (ap) val += ap[h] * static_cast<float>(kpos - qpos);
              }
              s[r * BK + c] = val;
            }
          }
          for (int64_t r = 0; r < rows; ++r) {
            float mx = mrow[r];
            for (int64_t c = 0; c < cols; ++c) mx = std::max(mx, s[r * BK + c]);
            if (mx == -INFINITY) continue;  // nothing visible in this block yet
            const float corr = std::exp(mrow[r] - mx);
            float sum = 0.0f;
            float* ar = acc.data() + r * D;
            for (int64_t e = 0; e < D; ++e) ar[e] *= corr;
            for (int64_t c = 0; c < cols; ++c) {
              const float pval = std::exp(s[r * BK + c] - mx);
              if (pval == 0.0f) continue;
              sum += pval;
              const float* vr = vp + ((b * Tk + k0 + c) * Hkv + hk) * D;
              for (int64_t e = 0; e < D; ++e) ar[e] += pval * vr[e];
            }
            lrow[r] = lrow[r] * corr + sum;
            mrow[r] = mx;
          }
        }
        for (int64_t r = 0; r < rows; ++r) {
          float* orow = op + ((b * Tq + q0 + r) * H + h) * D;
          const float inv = lrow[r] > 0.0f ? 1.0f / lrow[r] : 0.0f;
          for (int64_t e = 0; e < D; ++e) orow[e] = acc[r * D + e] * inv;
          lp[(b * H + h) * Tq + q0 + r] = lrow[r] > 0.0f ? mrow[r] + std::log(lrow[r]) : -INFINITY;
        }
      }
    });
  }
  return py::make_tuple(o, lse);
}

// INT8 weights with one scale per output row, or INT4 (two nibbles per byte, value = nibble - 8) with one
// scale per group; activations are quantised per row to INT8 first (integer dot products, exact).
struct PackedWeights {
  int bits = 8, group = 0;
  int64_t n = 0, k = 0;
  std::vector<int8_t> q8;
  std::vector<uint8_t> q4;
  std::vector<float> scales;
};

PackedWeights pack_weights(FArr w, int bits, int group) {
  if (w.ndim() != 2) throw std::invalid_argument("pack_weights: 2-D weights expected");
  PackedWeights p;
  p.bits = bits;
  p.n = w.shape(0);
  p.k = w.shape(1);
  const float* wp = w.data();
  if (bits == 8) {
    p.q8.resize(static_cast<size_t>(p.n * p.k));
    p.scales.resize(static_cast<size_t>(p.n));
    for (int64_t r = 0; r < p.n; ++r) {
      float am = 0;
      for (int64_t c = 0; c < p.k; ++c) am = std::max(am, std::fabs(wp[r * p.k + c]));
      const float s = am > 0 ? am / 127.0f : 1.0f;
      p.scales[static_cast<size_t>(r)] = s;
      for (int64_t c = 0; c < p.k; ++c)
        p.q8[static_cast<size_t>(r * p.k + c)] = static_cast<int8_t>(std::max(-127.0f, std::min(127.0f, std::nearbyint(wp[r * p.k + c] / s))));
    }
  } else if (bits == 4) {
    if (group <= 0 || p.k % group || group % 2) throw std::invalid_argument("pack_weights: bad group size");
    p.group = group;
    p.q4.resize(static_cast<size_t>(p.n * p.k / 2));
    p.scales.resize(static_cast<size_t>(p.n * (p.k / group)));
    for (int64_t r = 0; r < p.n; ++r)
      for (int64_t g = 0; g < p.k / group; ++g) {
        float am = 0;
        for (int j = 0; j < group; ++j) am = std::max(am, std::fabs(wp[r * p.k + g * group + j]));
        const float s = am > 0 ? am / 7.0f : 1.0f;
        p.scales[static_cast<size_t>(r * (p.k / group) + g)] = s;
        for (int j = 0; j < group; j += 2) {
          auto q = [&](int jj) {
            return static_cast<uint8_t>(std::max(-8.0f, std::min(7.0f, std::nearbyint(wp[r * p.k + g * group + jj] / s))) + 8);
          };
          p.q4[static_cast<size_t>((r * p.k + g * group + j) / 2)] = static_cast<uint8_t>(q(j) | (q(j + 1) << 4));
        }
      }
  } else {
    throw std::invalid_argument("pack_weights: bits must be 8 or 4");
  }
  return p;
}

py::array_t<float> cpu_quant_gemm(ThreadPool& pool, FArr x, const PackedWeights& p) {
  if (x.ndim() != 2 || x.shape(1) != p.k) throw std::invalid_argument("quant_gemm: shapes");
  const int64_t M = x.shape(0), K = p.k, N = p.n;
  std::vector<int8_t> xq(static_cast<size_t>(M * K));
  std::vector<float> xs(static_cast<size_t>(M));
  const float* xp = x.data();
  for (int64_t m = 0; m < M; ++m) {
    float am = 0;
    for (int64_t k = 0; k < K; ++k) am = std::max(am, std::fabs(xp[m * K + k]));
    const float s = am > 0 ? am / 127.0f : 1.0f;
    xs[static_cast<size_t>(m)] = s;
    for (int64_t k = 0; k < K; ++k)
      xq[static_cast<size_t>(m * K + k)] = static_cast<int8_t>(std::max(-127.0f, std::min(127.0f, std::nearbyint(xp[m * K + k] / s))));
  }
  py::array_t<float> y({M, N});
  float* yp = y.mutable_data();
  {
    py::gil_scoped_release rel;
    pool.run(N, [&](int, int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n)
        for (int64_t m = 0; m < M; ++m) {
          const int8_t* xr = xq.data() + m * K;
          float out = 0.0f;
          if (p.bits == 8) {
            const int8_t* wr = p.q8.data() + n * K;
            int32_t acc = 0;
            for (int64_t k = 0; k < K; ++k) acc += static_cast<int32_t>(xr[k]) * wr[k];
            out = static_cast<float>(acc) * p.scales[static_cast<size_t>(n)];
          } else {
            const int64_t groups = K / p.group;
            for (int64_t g = 0; g < groups; ++g) {
              int32_t acc = 0;
              for (int j = 0; j < p.group; ++j) {
                const int64_t k = g * p.group + j;
                const uint8_t b = p.q4[static_cast<size_t>((n * K + k) / 2)];
                const int q = static_cast<int>((b >> (4 * (k & 1))) & 15) - 8;
                acc += static_cast<int32_t>(xr[k]) * q;
              }
              out += static_cast<float>(acc) * p.scales[static_cast<size_t>(n * groups + g)];
            }
          }
          yp[m * N + n] = out * xs[static_cast<size_t>(m)];
        }
    });
  }
  return y;
}

}  // namespace

void bind_device_allocator(py::module_& m) {
  py::class_<DeviceCachingAllocator>(m, "DeviceCachingAllocator")
      .def(py::init<const std::string&, size_t>(), py::arg("backing") = "host", py::arg("limit_bytes") = 0)
      .def("alloc", &DeviceCachingAllocator::alloc, py::arg("bytes"), py::arg("stream") = 0)
      .def("free", &DeviceCachingAllocator::free)
      .def("record_stream", &DeviceCachingAllocator::record_stream)
      .def("empty_cache", &DeviceCachingAllocator::empty_cache)
      .def("stats", &DeviceCachingAllocator::stats);
  m.def("cpu_features", &cpu_features);
  py::class_<ThreadPool>(m, "ThreadPool")
      .def(py::init<int>(), py::arg("workers") = 0)
      .def_property_readonly("size", &ThreadPool::size)
      .def("partition", [](ThreadPool& p, int64_t n) {
        std::vector<std::tuple<int, int64_t, int64_t>> parts(static_cast<size_t>(p.size()), {-1, 0, 0});
        p.run(n, [&](int w, int64_t b, int64_t e) { parts[static_cast<size_t>(w)] = {w, b, e}; });
        return parts;
      });
  py::class_<PackedWeights>(m, "PackedWeights")
      .def_readonly("bits", &PackedWeights::bits)
      .def_readonly("group", &PackedWeights::group)
      .def_readonly("n", &PackedWeights::n)
      .def_readonly("k", &PackedWeights::k)
      .def_property_readonly("nbytes", [](const PackedWeights& p) {
        return p.q8.size() + p.q4.size() + p.scales.size() * sizeof(float);
      });
  m.def("pack_weights", &pack_weights, py::arg("w"), py::arg("bits") = 8, py::arg("group") = 32);
  m.def("cpu_gemm_nt", &cpu_gemm_nt, py::arg("pool"), py::arg("x"), py::arg("w"), py::arg("bias") = py::none());
  m.def("cpu_quant_gemm", &cpu_quant_gemm);
  m.def("cpu_gemm_nt_bf16", &cpu_gemm_nt_bf16, py::arg("pool"), py::arg("x"), py::arg("w"), py::arg("bias") = py::none());
  m.def("cpu_flash_attention", &cpu_flash_attention, py::arg("pool"), py::arg("q"), py::arg("k"), py::arg("v"),
        py::arg("causal") = true, py::arg("window") = 0, py::arg("scale") = 1.0, py::arg("softcap") = 0.0,
        py::arg("alibi") = FArr(0));
}
