// TCP key-value store for rendezvous and heartbeats (server and client) and the heartbeat analysis of the
// watchdog.  Wire format of a request: [u8 cmd][u32 key length][key][u64 value length][value]; of a reply:
// [u8 status][u64 length][payload]; little endian.  Commands: SET, GET (blocking, the value carries the timeout
// as a double), ADD (int64 delta, decimal value), CHECK, WAIT.  The server runs an accept thread and one thread
// per connection inside the process of rank 0; the client blocks without holding the interpreter lock.
// Parity: include/nexus/dist/store.hpp, src/dist/store.cpp and include/nexus/dist/watchdog.hpp:37-125 of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

enum : uint8_t { kSet = 1, kGet = 2, kAdd = 3, kCheck = 4, kWait = 5 };
enum : uint8_t { kOk = 0, kMissing = 1, kTimeout = 2 };

bool recv_exact(int fd, void* buf, size_t n) {
  auto* p = static_cast<uint8_t*>(buf);
  while (n > 0) {
    const ssize_t r = ::recv(fd, p, n, 0);
    if (r <= 0) return false;
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}
bool send_all(int fd, const void* buf, size_t n) {
  auto* p = static_cast<const uint8_t*>(buf);
  while (n > 0) {
    const ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
    if (r <= 0) return false;
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

class StoreServer {
 public:
  StoreServer(const std::string& host, int port) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) throw std::runtime_error("store: socket() failed");
    int one = 1;
    ::setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(port));
    if (::inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd_, 128) != 0) {
      ::close(fd_);
      throw std::runtime_error("store: cannot bind " + host + ":" + std::to_string(port));
    }
    socklen_t len = sizeof(addr);
    ::getsockname(fd_, reinterpret_cast<sockaddr*>(&addr), &len);
    port_ = ntohs(addr.sin_port);
    accept_ = std::thread([this] { accept_loop(); });
  }
  ~StoreServer() { shutdown(); }
  int port() const { return port_; }
  size_t keys() {
    std::lock_guard<std::mutex> g(mu_);
    return data_.size();
  }
  void shutdown() {
    if (stop_.exchange(true)) return;
    ::shutdown(fd_, SHUT_RDWR);
    ::close(fd_);
    {
      std::lock_guard<std::mutex> g(mu_);
      for (int c : conns_) ::shutdown(c, SHUT_RDWR);
    }
    cv_.notify_all();
    if (accept_.joinable()) accept_.join();
    for (auto& t : workers_)
      if (t.joinable()) t.join();
  }

 private:
  void accept_loop() {
    while (!stop_) {
      const int c = ::accept(fd_, nullptr, nullptr);
      if (c < 0) return;
      int one = 1;
      ::setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> g(mu_);
      conns_.push_back(c);
      workers_.emplace_back([this, c] { serve(c); });
    }
  }
  void reply(int c, uint8_t status, const std::string& payload = std::string()) {
    uint8_t head[9];
    head[0] = status;
    const uint64_t n = payload.size();
    std::memcpy(head + 1, &n, 8);
    if (send_all(c, head, 9) && n) send_all(c, payload.data(), n);
  }
  void serve(int c) {
    for (;;) {
      uint8_t head[5];
      if (!recv_exact(c, head, 5)) break;
      uint32_t klen;
      std::memcpy(&klen, head + 1, 4);
      std::string key(klen, '\0');
      if (klen && !recv_exact(c, key.data(), klen)) break;
      uint64_t vlen;
      if (!recv_exact(c, &vlen, 8) || vlen > (1ull << 32)) break;
      std::string val(vlen, '\0');
      if (vlen && !recv_exact(c, val.data(), vlen)) break;
      const uint8_t cmd = head[0];
      if (cmd == kSet) {
        {
          std::lock_guard<std::mutex> g(mu_);
          data_[key] = std::move(val);
        }
        cv_.notify_all();
        reply(c, kOk);
      } else if (cmd == kGet || cmd == kWait) {
        double timeout = 300.0;
        if (val.size() == 8) std::memcpy(&timeout, val.data(), 8);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout);
        std::unique_lock<std::mutex> g(mu_);
        const bool have = cv_.wait_until(g, deadline, [&] { return stop_.load() || data_.count(key) > 0; }) && data_.count(key);
        if (!have) {
          g.unlock();
          reply(c, kTimeout);
        } else {
          const std::string got = cmd == kGet ? data_[key] : std::string();
          g.unlock();
          reply(c, kOk, got);
        }
      } else if (cmd == kAdd) {
        int64_t delta = 0;
        if (val.size() == 8) std::memcpy(&delta, val.data(), 8);
        int64_t cur;
        {
          std::lock_guard<std::mutex> g(mu_);
          auto it = data_.find(key);
          cur = (it == data_.end() ? 0 : std::strtoll(it->second.c_str(), nullptr, 10)) + delta;
          data_[key] = std::to_string(cur);
        }
        cv_.notify_all();
        reply(c, kOk, std::string(reinterpret_cast<const char*>(&cur), 8));
      } else if (cmd == kCheck) {
        bool have;
        {
          std::lock_guard<std::mutex> g(mu_);
          have = data_.count(key) > 0;
        }
        reply(c, have ? kOk : kMissing);
      } else {
        break;
      }
    }
    ::close(c);
  }

  int fd_ = -1, port_ = 0;
  std::atomic<bool> stop_{false};
  std::thread accept_;
  std::vector<std::thread> workers_;
  std::vector<int> conns_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<std::string, std::string> data_;
};

class StoreClient {
 public:
  StoreClient(const std::string& host, int port, double timeout_s) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
    for (;;) {
      fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
      sockaddr_in addr{};
      addr.sin_family = AF_INET;
      addr.sin_port = htons(static_cast<uint16_t>(port));
      bool resolved = ::inet_pton(AF_INET, host.c_str(), &addr.sin_addr) == 1;
      if (!resolved) {
        addrinfo hints{}, *res = nullptr;
        hints.ai_family = AF_INET;
        hints.ai_socktype = SOCK_STREAM;
        if (::getaddrinfo(host.c_str(), nullptr, &hints, &res) == 0 && res != nullptr) {
          addr.sin_addr = reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr;
          ::freeaddrinfo(res);
          resolved = true;
        }
      }
      if (resolved && ::connect(fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) break;
      ::close(fd_);
      fd_ = -1;
      if (std::chrono::steady_clock::now() > deadline)
        throw std::runtime_error("no store at " + host + ":" + std::to_string(port));
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    int one = 1;
    ::setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  }
  ~StoreClient() { close(); }
  void close() {
    if (fd_ >= 0) {
      ::close(fd_);
      fd_ = -1;
    }
  }
  // one request / reply; the interpreter lock is released while the call blocks
  std::pair<int, py::bytes> call(int cmd, const std::string& key, const std::string& value) {
    uint8_t status = kTimeout;
    std::string payload;
    bool ok = true;
    {
      py::gil_scoped_release rel;
      std::lock_guard<std::mutex> g(mu_);
      std::string req(5 + key.size() + 8 + value.size(), '\0');
      req[0] = static_cast<char>(cmd);
      const uint32_t klen = static_cast<uint32_t>(key.size());
      std::memcpy(&req[1], &klen, 4);
      std::memcpy(&req[5], key.data(), key.size());
      const uint64_t vlen = value.size();
      std::memcpy(&req[5 + key.size()], &vlen, 8);
      std::memcpy(&req[13 + key.size()], value.data(), value.size());
      uint8_t head[9];
      ok = fd_ >= 0 && send_all(fd_, req.data(), req.size()) && recv_exact(fd_, head, 9);
      if (ok) {
        status = head[0];
        uint64_t n;
        std::memcpy(&n, head + 1, 8);
        payload.resize(n);
        ok = n == 0 || recv_exact(fd_, payload.data(), n);
      }
    }
    if (!ok) throw std::runtime_error("store connection closed");
    return {static_cast<int>(status), py::bytes(payload)};
  }

 private:
  int fd_ = -1;
  std::mutex mu_;
};

// ------------------------------------------------------------------------------------------------
// Watchdog analysis: one pass over the ranks' last heartbeats (step, step milliseconds, wall-clock time).
// Returns (kind, rank, step, detail) tuples: "stalled" = behind the leader and silent for longer than the
// timeout (or never seen); "straggler" = arrived at a step later than `fraction` of the median step time
// (at least `min_lag`) after the first rank.  `arrivals` is the caller's window of complete steps.
// ------------------------------------------------------------------------------------------------
py::list watchdog_scan(const std::vector<py::object>& recs, double now, double stall_timeout, double fraction,
                       double min_lag, py::dict arrivals, int window) {
  struct Rec {
    bool live = false;
    long step = -1;
    double ms = 0, t = 0;
  };
  const int world = static_cast<int>(recs.size());
  std::vector<Rec> r(world);
  long leader = -1;
  bool any = false;
  for (int i = 0; i < world; ++i) {
    if (recs[i].is_none()) continue;
    py::dict d = recs[i].cast<py::dict>();
    r[i].live = true;
    r[i].step = d["step"].cast<long>();
    r[i].ms = d["ms"].cast<double>();
    r[i].t = d["t"].cast<double>();
    leader = std::max(leader, r[i].step);
    any = true;
  }
  py::list out;
  if (!any) return out;
  for (int i = 0; i < world; ++i)
    if (r[i].step < leader && (!r[i].live || now - r[i].t > stall_timeout))
      out.append(py::make_tuple("stalled", i, r[i].step, r[i].live ? now - r[i].t : 0.0));
  std::vector<double> durations;
  for (int i = 0; i < world; ++i) {
    if (!r[i].live) continue;
    py::object key = py::int_(r[i].step);
    if (!arrivals.contains(key)) arrivals[key] = py::dict();
    arrivals[key].cast<py::dict>()[py::int_(i)] = r[i].t;
    if (r[i].ms > 0) durations.push_back(r[i].ms / 1e3);
  }
  double med = 0.0;
  if (!durations.empty()) {
    std::sort(durations.begin(), durations.end());
    const size_t n = durations.size();
    med = n % 2 ? durations[n / 2] : 0.5 * (durations[n / 2 - 1] + durations[n / 2]);
  }
  const double thr = std::max(min_lag, fraction * med);
  std::vector<long> steps;
  for (auto item : arrivals) steps.push_back(item.first.cast<long>());
  std::sort(steps.begin(), steps.end());
  for (long s : steps) {
    py::dict arr = arrivals[py::int_(s)].cast<py::dict>();
    if (static_cast<int>(arr.size()) < world) continue;
    double first = 1e300;
    for (auto it : arr) first = std::min(first, it.second.cast<double>());
    for (auto it : arr) {
      const double t = it.second.cast<double>();
      if (t - first > thr) out.append(py::make_tuple("straggler", it.first.cast<int>(), s, t - first));
    }
  }
  const int drop = static_cast<int>(steps.size()) - window;
  for (int i = 0; i < drop; ++i) arrivals.attr("pop")(py::int_(steps[i]));
  return out;
}

}  // namespace

void bind_store(py::module_& m) {
  py::class_<StoreServer>(m, "StoreServer")
      .def(py::init<const std::string&, int>(), py::arg("host"), py::arg("port"))
      .def_property_readonly("port", &StoreServer::port)
      .def("keys", &StoreServer::keys)
      .def("shutdown", &StoreServer::shutdown, py::call_guard<py::gil_scoped_release>());
  py::class_<StoreClient>(m, "StoreClient")
      .def(py::init<const std::string&, int, double>(), py::arg("host"), py::arg("port"), py::arg("timeout_s"),
           py::call_guard<py::gil_scoped_release>())
      .def("call", &StoreClient::call, py::arg("cmd"), py::arg("key"), py::arg("value") = std::string())
      .def("close", &StoreClient::close);
  m.def("watchdog_scan", &watchdog_scan, py::arg("records"), py::arg("now"), py::arg("stall_timeout"),
        py::arg("fraction"), py::arg("min_lag"), py::arg("arrivals"), py::arg("window"));
}
