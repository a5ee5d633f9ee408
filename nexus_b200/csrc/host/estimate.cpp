// Analytic model of an LM training step (parameters, FLOPs, memory per GPU, roofline step time) and the
// auto-parallel search over (dp, tp, pp, cp, ZeRO stage, micro batch, recompute) under a per-GPU memory limit.
// The Python tool (`tools/estimate.py`) holds the command line and the dataclasses; the arithmetic and the search
// run here.  Inputs and outputs are plain dicts keyed by the dataclass field names.
// Parity: tools/nexus_estimate/{estimate,autoparallel}.{hpp,cpp} of the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cmath>
#include <tuple>
#include <vector>

namespace py = pybind11;

namespace {

struct Model {
  long n_layer, d_model, n_head, n_kv_head, d_ff, vocab, seq_len, micro_batch, learned_pos, gradient_accum;
  bool tie_head, ffn_swiglu, bias, rmsnorm;
};
struct DType { double param_bytes, grad_bytes, optim_bytes, master_bytes, activation_elem_bytes; };
struct Plan { long dp, tp, pp, cp, zero_stage; bool full_recompute, flash_attention, sequence_parallel; };
struct Cluster { long gpus, gpus_per_node; double mem_gib, peak_tflops, intra_gbps, inter_gbps, mfu, dp_overlap, reserve_gib; };

template <typename T>
T get(const py::dict& d, const char* k, T def) { return d.contains(k) ? d[k].cast<T>() : def; }

Model model_of(const py::dict& d) {
  return {get<long>(d, "n_layer", 12), get<long>(d, "d_model", 768), get<long>(d, "n_head", 12), get<long>(d, "n_kv_head", 12),
          get<long>(d, "d_ff", 3072), get<long>(d, "vocab", 50257), get<long>(d, "seq_len", 1024), get<long>(d, "micro_batch", 1),
          get<long>(d, "learned_pos", 0), get<long>(d, "gradient_accum", 1), get<bool>(d, "tie_head", true),
          get<bool>(d, "ffn_swiglu", false), get<bool>(d, "bias", true), get<bool>(d, "rmsnorm", false)};
}
DType dtype_of(const py::dict& d) {
  return {get<double>(d, "param_bytes", 2), get<double>(d, "grad_bytes", 4), get<double>(d, "optim_bytes", 8),
          get<double>(d, "master_bytes", 4), get<double>(d, "activation_elem_bytes", 2)};
}
Plan plan_of(const py::dict& d) {
  return {get<long>(d, "dp", 1), get<long>(d, "tp", 1), get<long>(d, "pp", 1), get<long>(d, "cp", 1), get<long>(d, "zero_stage", 0),
          get<bool>(d, "full_recompute", false), get<bool>(d, "flash_attention", true), get<bool>(d, "sequence_parallel", true)};
}
Cluster cluster_of(const py::dict& d) {
  return {get<long>(d, "gpus", 8), get<long>(d, "gpus_per_node", 8), get<double>(d, "mem_gib", 180.0),
          get<double>(d, "peak_tflops", 1390.0), get<double>(d, "intra_gbps", 725.0), get<double>(d, "inter_gbps", 50.0),
          get<double>(d, "mfu", 0.55), get<double>(d, "dp_overlap", 0.7), get<double>(d, "reserve_gib", 4.0)};
}

struct Params { double embedding, per_layer, attention, ffn, norms, head, final_norm, total; };

Params params(const Model& m) {
  const double d = static_cast<double>(m.d_model), hd = static_cast<double>(m.d_model / m.n_head);
  const double qkv_cols = (m.n_head + 2 * m.n_kv_head) * hd;
  const double qkv = d * qkv_cols + (m.bias ? qkv_cols : 0.0);
  const double proj = d * d + (m.bias ? d : 0.0);
  const double ffn = (m.ffn_swiglu ? 3.0 : 2.0) * d * m.d_ff + (m.bias ? m.d_ff + d : 0.0);
  const double norms = 2.0 * d * (m.rmsnorm ? 1.0 : 2.0);
  Params p;
  p.attention = qkv + proj;
  p.ffn = ffn;
  p.norms = norms;
  p.per_layer = qkv + proj + ffn + norms;
  p.embedding = static_cast<double>(m.vocab) * d + static_cast<double>(m.learned_pos) * d;
  p.head = m.tie_head ? 0.0 : static_cast<double>(m.vocab) * d;
  p.final_norm = d * (m.rmsnorm ? 1.0 : 2.0);
  p.total = m.n_layer * p.per_layer + p.embedding + p.head + p.final_norm;
  return p;
}

double flops_per_token(const Model& m, bool causal) {
  const Params p = params(m);
  const double matrix = p.total - p.embedding + (m.tie_head ? static_cast<double>(m.vocab) * m.d_model : 0.0);
  const double attn = 12.0 * m.n_layer * m.d_model * m.seq_len * (causal ? 0.5 : 1.0);
  return 6.0 * matrix + attn;
}

struct Memory { double params, grads, optimizer, activations, logits, stat, total; };

Memory memory(const Model& m, const DType& dt, const Plan& pl) {
  const double n = params(m).total / static_cast<double>(pl.tp * pl.pp);
  const long z = pl.zero_stage;
  Memory r;
  r.params = n * dt.param_bytes / (z >= 3 ? pl.dp : 1);
  r.grads = n * dt.grad_bytes / (z >= 2 ? pl.dp : 1);
  r.optimizer = n * (dt.optim_bytes + dt.master_bytes) / (z >= 1 ? pl.dp : 1);
  const double s = static_cast<double>(m.seq_len) / pl.cp, b = static_cast<double>(m.micro_batch), h = static_cast<double>(m.d_model),
               a = static_cast<double>(m.n_head);
  const double e = dt.activation_elem_bytes / 2.0;
  double per_layer;
  if (pl.full_recompute) {
    per_layer = 2 * s * b * h * e;
  } else {
    per_layer = s * b * h * (34 + (pl.flash_attention ? 0.0 : 5 * a * s * pl.cp / h)) * e;
    if (pl.tp > 1) per_layer = pl.sequence_parallel ? per_layer / pl.tp : (10 + 24.0 / pl.tp) / 34 * per_layer;
  }
  const double layers = static_cast<double>(m.n_layer) / pl.pp;
  const double in_flight = pl.pp > 1 ? static_cast<double>(std::min<long>(pl.pp, std::max<long>(1, m.gradient_accum))) : 1.0;
  r.activations = per_layer * layers * in_flight;
  r.logits = s * b * (static_cast<double>(m.vocab) / pl.tp) * (dt.activation_elem_bytes + 4);
  r.stat = r.params + r.grads + r.optimizer;
  r.total = r.stat + r.activations + r.logits;
  return r;
}

struct Time { double tokens, model_flops, compute_s, tp_comm_s, cp_comm_s, dp_comm_s, bubble, step_s, tokens_per_s, mfu; };

Time step_time(const Model& m, const Plan& pl, const Cluster& cl, const DType& dt) {
  Time t;
  t.tokens = static_cast<double>(m.micro_batch) * m.seq_len * m.gradient_accum * pl.dp;
  t.model_flops = flops_per_token(m, true) * t.tokens;
  const long gpus = pl.dp * pl.tp * pl.pp * pl.cp;
  const double recompute = pl.full_recompute ? 4.0 / 3.0 : 1.0;
  t.compute_s = t.model_flops * recompute / (gpus * cl.peak_tflops * 1e12 * cl.mfu);
  auto bw = [&](long group) { return (group <= cl.gpus_per_node ? cl.intra_gbps : cl.inter_gbps) * 1e9; };
  const double per_rank_tokens = static_cast<double>(m.micro_batch) * m.seq_len / pl.cp * m.gradient_accum;
  t.tp_comm_s = 0.0;
  if (pl.tp > 1) {
    const double vol = 4 * 2 * (static_cast<double>(m.n_layer) / pl.pp) * per_rank_tokens * m.d_model * dt.activation_elem_bytes;
    t.tp_comm_s = vol * 2 * (pl.tp - 1) / pl.tp / bw(pl.tp);
  }
  t.cp_comm_s = 0.0;
  if (pl.cp > 1) {
    const double kv = 2 * per_rank_tokens * (static_cast<double>(m.d_model) * m.n_kv_head / m.n_head) * dt.activation_elem_bytes;
    t.cp_comm_s = 0.3 * 3 * (static_cast<double>(m.n_layer) / pl.pp) * kv * (pl.cp - 1) / bw(pl.tp * pl.cp);
  }
  t.dp_comm_s = 0.0;
  if (pl.dp > 1) {
    const double n = params(m).total / static_cast<double>(pl.tp * pl.pp);
    const double vol = n * dt.grad_bytes * 2 * (pl.dp - 1) / pl.dp + (pl.zero_stage >= 3 ? n * dt.param_bytes : 0.0);
    t.dp_comm_s = (1 - cl.dp_overlap) * vol / bw(gpus);
  }
  t.bubble = pl.pp > 1 ? static_cast<double>(pl.pp - 1) / (m.gradient_accum + pl.pp - 1) : 0.0;
  t.step_s = (t.compute_s + t.tp_comm_s + t.cp_comm_s) / (1 - t.bubble) + t.dp_comm_s;
  t.tokens_per_s = t.tokens / t.step_s;
  t.mfu = t.model_flops / (t.step_s * gpus * cl.peak_tflops * 1e12);
  return t;
}

struct Candidate {
  long dp, tp, pp, cp, zero, micro_batch, accum;
  double memory_gib, static_gib, activation_gib, logits_gib, compute_s, tp_comm_s, cp_comm_s, dp_comm_s, bubble, step_s, mfu;
  bool fits, recompute;
};

Candidate evaluate(Model m, const Cluster& cl, long dp, long tp, long pp, long cp, long zero, long micro, long accum,
                   bool recompute, const DType& dt) {
  m.micro_batch = micro;
  m.gradient_accum = accum;
  const Plan pl{dp, tp, pp, cp, zero, recompute, true, true};
  const Memory mem = memory(m, dt, pl);
  const Time t = step_time(m, pl, cl, dt);
  const double gib = 1073741824.0;
  Candidate c{dp, tp, pp, cp, zero, micro, accum, mem.total / gib, mem.stat / gib, mem.activations / gib, mem.logits / gib,
              t.compute_s, t.tp_comm_s, t.cp_comm_s, t.dp_comm_s, t.bubble, t.step_s, t.mfu, false, recompute};
  c.fits = c.memory_gib + cl.reserve_gib <= cl.mem_gib;
  return c;
}

py::dict to_dict(const Candidate& c) {
  py::dict d;
  d["dp"] = c.dp; d["tp"] = c.tp; d["pp"] = c.pp; d["cp"] = c.cp; d["zero"] = c.zero; d["micro_batch"] = c.micro_batch;
  d["accum"] = c.accum; d["memory_gib"] = c.memory_gib; d["static_gib"] = c.static_gib; d["activation_gib"] = c.activation_gib;
  d["logits_gib"] = c.logits_gib; d["compute_s"] = c.compute_s; d["tp_comm_s"] = c.tp_comm_s; d["cp_comm_s"] = c.cp_comm_s;
  d["dp_comm_s"] = c.dp_comm_s; d["bubble"] = c.bubble; d["step_s"] = c.step_s; d["mfu"] = c.mfu; d["fits"] = c.fits;
  d["recompute"] = c.recompute;
  return d;
}

py::dict py_params(const py::dict& md) {
  const Params p = params(model_of(md));
  py::dict d;
  auto put = [&](const char* k, double v) { d[k] = static_cast<long long>(std::llround(v)); };
  put("embedding", p.embedding); put("per_layer", p.per_layer); put("attention", p.attention); put("ffn", p.ffn);
  put("norms", p.norms); put("head", p.head); put("final_norm", p.final_norm); put("total", p.total);
  return d;
}

py::dict py_memory(const py::dict& md, const py::dict& dtd, const py::dict& pld) {
  const Memory r = memory(model_of(md), dtype_of(dtd), plan_of(pld));
  py::dict d;
  d["params"] = r.params; d["grads"] = r.grads; d["optimizer"] = r.optimizer; d["activations"] = r.activations;
  d["logits"] = r.logits; d["static"] = r.stat; d["total"] = r.total;
  return d;
}

py::dict py_step_time(const py::dict& md, const py::dict& pld, const py::dict& cld, const py::dict& dtd) {
  const Time t = step_time(model_of(md), plan_of(pld), cluster_of(cld), dtype_of(dtd));
  py::dict d;
  d["tokens"] = static_cast<long long>(std::llround(t.tokens)); d["model_flops"] = t.model_flops; d["compute_s"] = t.compute_s;
  d["tp_comm_s"] = t.tp_comm_s; d["cp_comm_s"] = t.cp_comm_s; d["dp_comm_s"] = t.dp_comm_s; d["bubble"] = t.bubble;
  d["step_s"] = t.step_s; d["tokens_per_s"] = t.tokens_per_s; d["mfu"] = t.mfu;
  return d;
}

py::dict py_evaluate(const py::dict& md, const py::dict& cld, long dp, long tp, long pp, long cp, long zero, long micro,
                     long accum, bool recompute, const py::dict& dtd) {
  return to_dict(evaluate(model_of(md), cluster_of(cld), dp, tp, pp, cp, zero, micro, accum, recompute, dtype_of(dtd)));
}

// Exhaustive search over factorizations of the GPU count; the layouts that fit are ranked by step time, then by the
// model-parallel degree, then by the ZeRO stage.
py::dict py_auto_parallel(const py::dict& md, const py::dict& cld, long global_batch, long max_tp, long max_pp, long max_cp,
                          long top, const std::vector<long>& micro_batches, const py::dict& dtd) {
  const Model m = model_of(md);
  const Cluster cl = cluster_of(cld);
  const DType dt = dtype_of(dtd);
  auto divisors = [](long n) {
    std::vector<long> v;
    for (long i = 1; i <= n; ++i)
      if (n % i == 0) v.push_back(i);
    return v;
  };
  std::vector<Candidate> cands;
  long tried = 0;
  for (long tp : divisors(cl.gpus)) {
    if (tp > max_tp || m.n_head % tp || tp > cl.gpus_per_node) continue;
    for (long pp : divisors(cl.gpus / tp)) {
      if (pp > max_pp || m.n_layer % pp) continue;
      for (long cp : divisors(cl.gpus / (tp * pp))) {
        if (cp > max_cp || m.seq_len % (2 * cp)) continue;
        const long dp = cl.gpus / (tp * pp * cp);
        if (global_batch % dp) continue;
        const long per_dp = global_batch / dp;
        for (long micro : micro_batches) {
          if (per_dp % micro) continue;
          const long accum = per_dp / micro;
          const int zmax = dp > 1 ? 3 : 0;
          for (int zero = 0; zero <= zmax; ++zero)
            for (int rec = 0; rec < 2; ++rec) {
              ++tried;
              const Candidate c = evaluate(m, cl, dp, tp, pp, cp, zero, micro, accum, rec != 0, dt);
              if (c.fits) cands.push_back(c);
            }
        }
      }
    }
  }
  std::stable_sort(cands.begin(), cands.end(), [](const Candidate& a, const Candidate& b) {
    return std::make_tuple(a.step_s, a.tp * a.pp * a.cp, a.zero) < std::make_tuple(b.step_s, b.tp * b.pp * b.cp, b.zero);
  });
  py::list best;
  for (size_t i = 0; i < cands.size() && static_cast<long>(i) < top; ++i) best.append(to_dict(cands[i]));
  py::dict out;
  out["tried"] = tried;
  out["feasible"] = static_cast<long>(cands.size());
  out["best"] = best;
  return out;
}

}  // namespace

void bind_estimate(py::module_& m) {
  m.def("estimate_params", &py_params);
  m.def("estimate_flops_per_token", [](const py::dict& md, bool causal) { return flops_per_token(model_of(md), causal); },
        py::arg("model"), py::arg("causal") = true);
  m.def("estimate_memory", &py_memory);
  m.def("estimate_step_time", &py_step_time);
  m.def("estimate_evaluate", &py_evaluate);
  m.def("estimate_auto_parallel", &py_auto_parallel);
}
