// Driver for the reference arm of bench.py: trains GPT-2 124M with the reference's own, unmodified
// single-GPU path (nexus::cuda::GptModel + nexus::cuda::GptTrainer, cuBLASLt GEMMs and its
// FlashAttention-2 kernels) and prints one JSON line with the timings.  Nothing of nexus_b200 is
// linked here; the reference sources are compiled as they are by baseline/build_ref.py.
//
// C entry points (bench.py loads the shared library with ctypes; -DREF_DRIVER_MAIN adds a command line):
//   nexus_ref_gpt_open(batch, seq, tuned, autotune)   build model + optimizer config, returns 0 / error code
//   nexus_ref_gpt_device(steps, warmup, &ms, &loss)   device-timed region
//   nexus_ref_gpt_e2e(steps, warmup, &ms, &loss)      end-to-end region
//   nexus_ref_gpt_info(out, len)                      JSON description;  nexus_ref_gpt_close()
//
// Two timed regions, same steps / warm-up:
//   device : tokens already on the GPU, forward_backward + optimizer_step per step, CUDA events
//   e2e    : GptTrainer::step(host tokens) with a loss read every step, i.e. the pinned host -> device
//            copy of the tokens and the device -> host read of the loss are inside the region
#include "nexus/cuda/caching_allocator.hpp"
#include "nexus/cuda/gemm.hpp"
#include "nexus/cuda/gpt.hpp"
#include "nexus/cuda/runtime.hpp"

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <vector>

namespace nc = nexus::cuda;

namespace {
struct State {
  nc::Stream stream;
  std::unique_ptr<nc::StreamGuard> guard;
  std::unique_ptr<nc::GptModel> model;
  nc::DeviceAdamWConfig adam;
  std::vector<std::vector<std::int32_t>> host;
  std::size_t count = 0;
  int batch = 0, seq = 0, tuned = 0, autotune = 0;
};
std::unique_ptr<State> g_state;
std::string g_error;

int fail(const std::exception& e) {
  g_error = e.what();
  for (auto& c : g_error)
    if (c == '"' || c == '\n' || c == '\\') c = ' ';
  return 2;
}
constexpr int kSets = 4;
}  // namespace

extern "C" const char* nexus_ref_gpt_error() { return g_error.c_str(); }

extern "C" int nexus_ref_gpt_open(int batch, int seq, int tuned, int autotune) {
  try {
    if (nc::device_count() == 0) {
      g_error = "no CUDA device";
      return 77;
    }
    auto st = std::make_unique<State>();
    nc::set_float32_matmul_precision(nc::MatmulPrecision::High);
    if (autotune) nc::set_gemm_autotune(true);
    nc::GptConfig config;  // GPT-2 124M: vocab 50257, 12 layers, 12 heads, dim 768, max_seq 1024
    config.max_seq = seq > 1024 ? seq : 1024;
    config.compute_dtype = nexus::DType::BF16;
    config.master = nc::MasterWeights::Fp32Master;
    config.attention = nc::AttentionBackend::Flash;
    config.optimizer = nc::OptimizerKind::AdamW;
    config.recompute = nc::Recompute::None;
    config.ce_chunk_rows = 0;
    if (tuned) {  // what the reference's own compile(true) mode switches on (lm_backend.cpp:76-78)
      config.vocab_pad_multiple = 64;
      config.fuse_ce_cast = true;
      config.fast_ce = true;
    }
    st->stream = nc::Stream::create(0);
    st->guard = std::make_unique<nc::StreamGuard>(st->stream);
    st->model = std::make_unique<nc::GptModel>(config, batch, seq, 1337, st->stream);
    st->adam.lr = 6.0e-4;
    st->adam.beta1 = 0.9;
    st->adam.beta2 = 0.95;
    st->adam.eps = 1.0e-8;
    st->adam.weight_decay = 0.1;
    st->adam.max_grad_norm = 1.0;
    st->count = static_cast<std::size_t>(batch) * seq;
    std::mt19937 rng(1234);
    std::uniform_int_distribution<int> token(0, config.vocab - 1);
    st->host.assign(kSets, std::vector<std::int32_t>(st->count));
    for (auto& h : st->host)
      for (auto& t : h) t = token(rng);
    st->batch = batch;
    st->seq = seq;
    st->tuned = tuned;
    st->autotune = autotune;
    g_state = std::move(st);
    return 0;
  } catch (const std::exception& e) {
    return fail(e);
  }
}

// Tokens resident on the device; K x (forward_backward + optimizer_step) between two CUDA events.
extern "C" int nexus_ref_gpt_device(int steps, int warmup, double* ms_per_step, float* loss) {
  try {
    State& st = *g_state;
    nc::DeviceBuffer d_tokens[kSets];
    for (int i = 0; i < kSets; ++i) {
      d_tokens[i] = nc::DeviceBuffer(st.count * sizeof(std::int32_t), st.stream);
      NEXUS_CUDA_CHECK(cudaMemcpyAsync(d_tokens[i].data(), st.host[i].data(), st.count * 4, cudaMemcpyHostToDevice,
                                       st.stream.handle()));
    }
    for (int i = 0; i < warmup; ++i) {
      st.model->forward_backward(d_tokens[i % kSets].as<std::int32_t>());
      st.model->optimizer_step(st.adam);
    }
    st.stream.synchronize();
    nc::Event begin, end;
    begin.record(st.stream);
    for (int i = 0; i < steps; ++i) {
      st.model->forward_backward(d_tokens[i % kSets].as<std::int32_t>());
      st.model->optimizer_step(st.adam);
    }
    end.record(st.stream);
    end.synchronize();
    *ms_per_step = begin.elapsed_ms(end) / steps;
    *loss = st.model->read_loss();
    return std::isfinite(*loss) ? 0 : 3;
  } catch (const std::exception& e) {
    return fail(e);
  }
}

// The reference's trainer: host tokens in (pinned double buffer, H2D inside), loss read back every step.
extern "C" int nexus_ref_gpt_e2e(int steps, int warmup, double* ms_per_step, float* loss) {
  try {
    State& st = *g_state;
    nc::GptTrainer trainer(*st.model, st.adam, /*loss_read_interval=*/1);
    for (int i = 0; i < warmup; ++i) trainer.step(st.host[i % kSets].data());
    trainer.synchronize();
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) trainer.step(st.host[i % kSets].data());
    *loss = trainer.synchronize();
    const auto t1 = std::chrono::steady_clock::now();
    *ms_per_step = std::chrono::duration<double, std::milli>(t1 - t0).count() / steps;
    return std::isfinite(*loss) ? 0 : 3;
  } catch (const std::exception& e) {
    return fail(e);
  }
}

extern "C" int nexus_ref_gpt_info(char* out, int out_len) {
  try {
    State& st = *g_state;
    const auto stats = nc::caching_device_allocator().stats(0);
    std::snprintf(out, out_len,
                  "{\"batch\": %d, \"seq\": %d, \"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": 4, "
                  "\"attention\": \"%s\", \"parameters\": %zu, \"peak_reserved_bytes\": %zu, \"tuned\": %d, "
                  "\"autotune\": %d}",
                  st.batch, st.seq, st.count * 4, nc::to_string(st.model->attention_backend()),
                  st.model->num_parameters(), static_cast<std::size_t>(stats.peak_reserved_bytes), st.tuned,
                  st.autotune);
    return 0;
  } catch (const std::exception& e) {
    return fail(e);
  }
}

extern "C" void nexus_ref_gpt_close() { g_state.reset(); }

#ifdef REF_DRIVER_MAIN
namespace {
int arg_int(int argc, char** argv, const char* key, int fallback) {
  for (int i = 1; i + 1 < argc; ++i)
    if (std::strcmp(argv[i], key) == 0) return std::atoi(argv[i + 1]);
  return fallback;
}
}  // namespace

int main(int argc, char** argv) {
  const int steps = arg_int(argc, argv, "--steps", 20), warmup = arg_int(argc, argv, "--warmup", 5);
  int rc = nexus_ref_gpt_open(arg_int(argc, argv, "--batch", 16), arg_int(argc, argv, "--seq", 1024),
                              arg_int(argc, argv, "--tuned", 1), arg_int(argc, argv, "--autotune", 0));
  double dev = 0, e2e = 0;
  float l0 = 0, l1 = 0;
  if (rc == 0) rc = nexus_ref_gpt_device(steps, warmup, &dev, &l0);
  if (rc == 0) rc = nexus_ref_gpt_e2e(steps, warmup, &e2e, &l1);
  if (rc != 0) {
    std::printf("{\"error\": \"%s\", \"rc\": %d}\n", nexus_ref_gpt_error(), rc);
    return rc;
  }
  static char info[2048];
  nexus_ref_gpt_info(info, sizeof(info));
  std::printf("{\"device_ms_per_step\": %.5f, \"e2e_ms_per_step\": %.5f, \"device_loss\": %.5f, \"e2e_loss\": %.5f, "
              "\"info\": %s}\n", dev, e2e, l0, l1, info);
  nexus_ref_gpt_close();
  return 0;
}
#endif
