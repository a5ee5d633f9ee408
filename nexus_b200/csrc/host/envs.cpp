// Native reinforcement-learning environments (LineWorld, GridWorld, CartPole, PointMass) and a
// vectorised runner with persistent worker threads that steps N environments per call and
// auto-resets finished episodes.
// Parity: include/nexus/rl/envs.hpp:33-240 and include/nexus/rl/vector_env.hpp of the reference
// (same dynamics, rewards, horizons and termination rules).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

struct Step {
  std::vector<float> obs;
  float reward = 0.0f;
  bool terminated = false;
  bool truncated = false;
};

class Env {
 public:
  virtual ~Env() = default;
  virtual int obs_dim() const = 0;
  virtual int action_count() const = 0;  // discrete: number of actions; continuous: dimension
  virtual bool discrete() const = 0;
  virtual std::vector<float> reset(uint32_t seed) = 0;
  virtual Step step(const float* action) = 0;
};

std::vector<float> one_hot(int i, int n) {
  std::vector<float> v(static_cast<size_t>(n), 0.0f);
  v[static_cast<size_t>(i)] = 1.0f;
  return v;
}

int read_discrete(const float* a, int n) {
  const int c = static_cast<int>(std::lround(a[0]));
  if (c < 0 || c >= n) throw std::invalid_argument("discrete action out of range");
  return c;
}

class LineWorld final : public Env {
 public:
  LineWorld(int length, int horizon) : length_(length), horizon_(horizon) {
    if (length < 2) throw std::invalid_argument("LineWorld length must be at least 2");
  }
  int obs_dim() const override { return length_; }
  int action_count() const override { return 2; }
  bool discrete() const override { return true; }
  std::vector<float> reset(uint32_t) override {
    pos_ = steps_ = 0;
    return one_hot(0, length_);
  }
  Step step(const float* a) override {
    const int c = read_discrete(a, 2);
    Step r;
    if (c == 1 && pos_ < length_ - 1) {
      ++pos_;
      r.reward = 0.1f;
    } else if (c == 0 && pos_ > 0) {
      --pos_;
    }
    ++steps_;
    if (pos_ == length_ - 1) {
      r.reward += 1.0f;
      r.terminated = true;
    } else if (steps_ >= horizon_) {
      r.truncated = true;
    }
    r.obs = one_hot(pos_, length_);
    return r;
  }

 private:
  int length_, horizon_, pos_ = 0, steps_ = 0;
};

class GridWorld final : public Env {
 public:
  GridWorld(int width, int horizon) : w_(width), horizon_(horizon) {}
  int obs_dim() const override { return w_ * w_; }
  int action_count() const override { return 4; }
  bool discrete() const override { return true; }
  std::vector<float> reset(uint32_t) override {
    row_ = col_ = steps_ = 0;
    return one_hot(0, w_ * w_);
  }
  Step step(const float* a) override {
    const int c = read_discrete(a, 4);
    if (c == 0 && col_ + 1 < w_) ++col_;
    else if (c == 1 && col_ > 0) --col_;
    else if (c == 2 && row_ + 1 < w_) ++row_;
    else if (c == 3 && row_ > 0) --row_;
    ++steps_;
    Step r;
    r.reward = -0.01f;
    if (row_ == w_ - 1 && col_ == w_ - 1) {
      r.reward = 1.0f;
      r.terminated = true;
    } else if (steps_ >= horizon_) {
      r.truncated = true;
    }
    r.obs = one_hot(row_ * w_ + col_, w_ * w_);
    return r;
  }

 private:
  int w_, horizon_, row_ = 0, col_ = 0, steps_ = 0;
};

struct SplitMix {
  uint64_t s;
  explicit SplitMix(uint64_t seed) : s(seed) {}
  float uniform() {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
  }
};

class CartPole final : public Env {
 public:
  int obs_dim() const override { return 4; }
  int action_count() const override { return 2; }
  bool discrete() const override { return true; }
  std::vector<float> reset(uint32_t seed) override {
    SplitMix rng(seed);
    x_ = (rng.uniform() - 0.5f) * 0.1f;
    xd_ = (rng.uniform() - 0.5f) * 0.1f;
    th_ = (rng.uniform() - 0.5f) * 0.1f;
    thd_ = (rng.uniform() - 0.5f) * 0.1f;
    steps_ = 0;
    return {x_, xd_, th_, thd_};
  }
  Step step(const float* a) override {
    const int c = read_discrete(a, 2);
    constexpr float g = 9.8f, mc = 1.0f, mp = 0.1f, total = mc + mp, len = 0.5f, pml = mp * len, fmag = 10.0f,
                    tau = 0.02f, th_lim = 12.0f * 3.14159265f / 180.0f, x_lim = 2.4f;
    const float force = c == 1 ? fmag : -fmag;
    const float ct = std::cos(th_), st = std::sin(th_);
    const float temp = (force + pml * thd_ * thd_ * st) / total;
    const float th_acc = (g * st - ct * temp) / (len * (4.0f / 3.0f - mp * ct * ct / total));
    const float x_acc = temp - pml * th_acc * ct / total;
    x_ += tau * xd_;
    xd_ += tau * x_acc;
    th_ += tau * thd_;
    thd_ += tau * th_acc;
    ++steps_;
    Step r;
    r.reward = 1.0f;
    r.terminated = std::fabs(x_) > x_lim || std::fabs(th_) > th_lim;
    r.truncated = steps_ >= 500;
    r.obs = {x_, xd_, th_, thd_};
    return r;
  }

 private:
  float x_ = 0, xd_ = 0, th_ = 0, thd_ = 0;
  int steps_ = 0;
};

class PointMass final : public Env {
 public:
  int obs_dim() const override { return 1; }
  int action_count() const override { return 1; }
  bool discrete() const override { return false; }
  std::vector<float> reset(uint32_t) override {
    x_ = 1.0f;
    steps_ = 0;
    return {x_};
  }
  Step step(const float* a) override {
    const float c = std::clamp(a[0], -1.0f, 1.0f);
    x_ = std::clamp(x_ + 0.5f * c, -2.0f, 2.0f);
    ++steps_;
    Step r;
    r.reward = -x_ * x_;
    r.truncated = steps_ >= 10;
    r.obs = {x_};
    return r;
  }

 private:
  float x_ = 1.0f;
  int steps_ = 0;
};

std::unique_ptr<Env> make_env(const std::string& kind, int a, int b) {
  if (kind == "LineWorld") return std::make_unique<LineWorld>(a > 0 ? a : 5, b > 0 ? b : 12);
  if (kind == "GridWorld") return std::make_unique<GridWorld>(a > 0 ? a : 4, b > 0 ? b : 24);
  if (kind == "CartPole") return std::make_unique<CartPole>();
  if (kind == "PointMass") return std::make_unique<PointMass>();
  throw std::invalid_argument("unknown environment: " + kind);
}

// Python-facing single environment.
class PyEnv {
 public:
  PyEnv(const std::string& kind, int a, int b) : env_(make_env(kind, a, b)), kind_(kind) {}
  py::array_t<float> reset(uint32_t seed) { return to_array(env_->reset(seed)); }
  py::tuple step(py::array_t<float, py::array::c_style | py::array::forcecast> action) {
    if (action.size() < 1) throw std::invalid_argument("empty action");
    Step s = env_->step(action.data());
    return py::make_tuple(to_array(s.obs), s.reward, s.terminated, s.truncated);
  }
  int obs_dim() const { return env_->obs_dim(); }
  int action_count() const { return env_->action_count(); }
  bool discrete() const { return env_->discrete(); }
  std::string kind() const { return kind_; }

 private:
  static py::array_t<float> to_array(const std::vector<float>& v) {
    py::array_t<float> a(static_cast<py::ssize_t>(v.size()));
    std::copy(v.begin(), v.end(), a.mutable_data());
    return a;
  }
  std::unique_ptr<Env> env_;
  std::string kind_;
};

// N environments stepped by persistent workers; finished episodes reset automatically (the returned
// observation is the first one of the next episode, flags describe the finished one).
class VectorEnv {
 public:
  VectorEnv(const std::string& kind, int count, int a, int b, int workers, uint32_t seed)
      : n_(count), seed_(seed) {
    if (count < 1) throw std::invalid_argument("VectorEnv needs at least one environment");
    for (int i = 0; i < count; ++i) envs_.push_back(make_env(kind, a, b));
    obs_dim_ = envs_[0]->obs_dim();
    act_dim_ = envs_[0]->discrete() ? 1 : envs_[0]->action_count();
    episodes_.assign(static_cast<size_t>(count), 0);
    const int nw = std::max(1, std::min(workers > 0 ? workers : static_cast<int>(std::thread::hardware_concurrency()),
                                        count));
    for (int w = 0; w < nw; ++w) threads_.emplace_back([this, w, nw] { worker(w, nw); });
  }
  ~VectorEnv() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
      ++generation_;
    }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  py::array_t<float> reset() {
    py::array_t<float> out({n_, obs_dim_});
    for (int i = 0; i < n_; ++i) {
      auto o = envs_[static_cast<size_t>(i)]->reset(seed_ + static_cast<uint32_t>(i));
      std::copy(o.begin(), o.end(), out.mutable_data() + static_cast<size_t>(i) * obs_dim_);
    }
    return out;
  }
  py::tuple step(py::array_t<float, py::array::c_style | py::array::forcecast> actions) {
    if (actions.size() != static_cast<py::ssize_t>(n_) * act_dim_) throw std::invalid_argument("bad action batch shape");
    py::array_t<float> obs({n_, obs_dim_});
    py::array_t<float> rew(n_);
    py::array_t<bool> term(n_), trunc(n_);
    a_ = actions.data();
    o_ = obs.mutable_data();
    r_ = rew.mutable_data();
    te_ = term.mutable_data();
    tr_ = trunc.mutable_data();
    {
      py::gil_scoped_release nogil;
      std::unique_lock<std::mutex> lk(mu_);
      pending_ = static_cast<int>(threads_.size());
      ++generation_;
      cv_.notify_all();
      done_cv_.wait(lk, [this] { return pending_ == 0; });
    }
    if (!error_.empty()) {
      std::string e = error_;
      error_.clear();
      throw std::runtime_error(e);
    }
    steps_ += n_;
    return py::make_tuple(obs, rew, term, trunc);
  }
  int size() const { return n_; }
  int obs_dim() const { return obs_dim_; }
  long long total_steps() const { return steps_; }

 private:
  void worker(int w, int nw) {
    uint64_t seen = 0;
    while (true) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return generation_ != seen; });
        seen = generation_;
        if (stop_) return;
      }
      try {
        for (int i = w; i < n_; i += nw) {
          Env& e = *envs_[static_cast<size_t>(i)];
          Step s = e.step(a_ + static_cast<size_t>(i) * act_dim_);
          r_[i] = s.reward;
          te_[i] = s.terminated;
          tr_[i] = s.truncated;
          if (s.terminated || s.truncated) {
            episodes_[static_cast<size_t>(i)] += 1;
            s.obs = e.reset(seed_ + static_cast<uint32_t>(i) + 7919u * static_cast<uint32_t>(episodes_[static_cast<size_t>(i)]));
          }
          std::copy(s.obs.begin(), s.obs.end(), o_ + static_cast<size_t>(i) * obs_dim_);
        }
      } catch (const std::exception& ex) {
        std::lock_guard<std::mutex> lk(mu_);
        error_ = ex.what();
      }
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (--pending_ == 0) done_cv_.notify_all();
      }
    }
  }
  int n_, obs_dim_ = 0, act_dim_ = 1;
  uint32_t seed_;
  std::vector<std::unique_ptr<Env>> envs_;
  std::vector<int> episodes_;
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  uint64_t generation_ = 0;
  int pending_ = 0;
  bool stop_ = false;
  std::string error_;
  const float* a_ = nullptr;
  float *o_ = nullptr, *r_ = nullptr;
  bool *te_ = nullptr, *tr_ = nullptr;
  long long steps_ = 0;
};

}  // namespace

void bind_envs(py::module_& m) {
  py::class_<PyEnv>(m, "NativeEnv")
      .def(py::init<const std::string&, int, int>(), py::arg("kind"), py::arg("a") = 0, py::arg("b") = 0)
      .def("reset", &PyEnv::reset, py::arg("seed") = 0)
      .def("step", &PyEnv::step)
      .def_property_readonly("obs_dim", &PyEnv::obs_dim)
      .def_property_readonly("action_count", &PyEnv::action_count)
      .def_property_readonly("discrete", &PyEnv::discrete)
      .def_property_readonly("kind", &PyEnv::kind);
  py::class_<VectorEnv>(m, "NativeVectorEnv")
      .def(py::init<const std::string&, int, int, int, int, uint32_t>(), py::arg("kind"), py::arg("count"),
           py::arg("a") = 0, py::arg("b") = 0, py::arg("workers") = 0, py::arg("seed") = 0)
      .def("reset", &VectorEnv::reset)
      .def("step", &VectorEnv::step)
      .def_property_readonly("size", &VectorEnv::size)
      .def_property_readonly("obs_dim", &VectorEnv::obs_dim)
      .def_property_readonly("total_steps", &VectorEnv::total_steps);
}
