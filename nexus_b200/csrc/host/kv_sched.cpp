// Host bookkeeping of the paged-KV inference engine: block pool with reference counts, per-sequence block lists and
// token lists, copy-on-write on append to a shared partial block, truncation, and the packing of one step's batch into
// the six index rows the device kernels read (token, position, cache slot, sequence, context length, logit rows).
// The engine calls `plan` with the step's chunks, picks a staging width from the result, and has `write` fill the
// (pinned) staging rows; block copies for copy-on-write and block-table rows of the sequences that changed are
// reported back for the engine to issue on the device.
// Parity: the sequence / block management and batch assembly of src/cuda/infer.cpp in the reference.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace py = pybind11;

namespace {

struct Seq {
  bool live = false;
  std::vector<int32_t> blocks;
  std::vector<int32_t> tokens;
  int length = 0;
  int n_prompt = 0;
};

class KvScheduler {
 public:
  KvScheduler(int n_blocks, int block_size, int max_seqs, int ctx)
      : bs_(block_size), ctx_(ctx), refcount_(static_cast<size_t>(n_blocks), 0), seqs_(static_cast<size_t>(max_seqs)) {
    if (n_blocks <= 0 || block_size <= 0 || max_seqs <= 0 || ctx <= 0) throw std::invalid_argument("KvScheduler: bad sizes");
    free_blocks_.reserve(static_cast<size_t>(n_blocks));
    for (int b = n_blocks - 1; b >= 0; --b) free_blocks_.push_back(b);
    for (int s = max_seqs - 1; s >= 0; --s) free_ids_.push_back(s);
  }

  int add() {
    if (free_ids_.empty()) throw std::runtime_error("no free sequence slot (max_seqs reached)");
    const int sid = free_ids_.back();
    free_ids_.pop_back();
    Seq& s = seqs_[static_cast<size_t>(sid)];
    s = Seq{};
    s.live = true;
    return sid;
  }

  int fork(int src) {
    (void)at(src);                                   // refuses an unknown source before a slot is taken
    const int sid = add();
    Seq& s = seqs_[static_cast<size_t>(sid)];
    const Seq& f = seqs_[static_cast<size_t>(src)];
    s.blocks = f.blocks;
    s.tokens = f.tokens;
    s.length = f.length;
    s.n_prompt = f.n_prompt;
    for (int32_t b : s.blocks) ++refcount_[static_cast<size_t>(b)];
    return sid;
  }

  void free(int sid) {
    Seq& s = at(sid);
    for (int32_t b : s.blocks) release(b);
    s = Seq{};
    free_ids_.push_back(sid);
  }

  // Shortens the sequence; returns the dropped tokens and how many of them were model output.
  py::tuple truncate(int sid, int length) {
    Seq& s = at(sid);
    if (length < 0 || length > s.length) throw std::invalid_argument("truncate: bad length");
    std::vector<int32_t> removed;
    if (length == s.length) return py::make_tuple(removed, 0);
    const size_t keep = static_cast<size_t>((length + bs_ - 1) / bs_);
    for (size_t i = keep; i < s.blocks.size(); ++i) release(s.blocks[i]);
    s.blocks.resize(keep);
    removed.assign(s.tokens.begin() + length, s.tokens.end());
    s.tokens.resize(static_cast<size_t>(length));
    const int n_out = s.length - std::max(s.n_prompt, length);
    s.length = length;
    s.n_prompt = std::min(s.n_prompt, length);
    return py::make_tuple(removed, std::max(0, n_out));
  }

  bool live(int sid) const { return sid >= 0 && static_cast<size_t>(sid) < seqs_.size() && seqs_[static_cast<size_t>(sid)].live; }
  int length(int sid) const { return at(sid).length; }
  int n_prompt(int sid) const { return at(sid).n_prompt; }
  std::vector<int32_t> tokens(int sid) const { return at(sid).tokens; }
  std::vector<int32_t> blocks(int sid) const { return at(sid).blocks; }
  int refcount(int block) const { return refcount_.at(static_cast<size_t>(block)); }
  int free_blocks() const { return static_cast<int>(free_blocks_.size()); }
  int total_blocks() const { return static_cast<int>(refcount_.size()); }
  int live_sequences() const { return static_cast<int>(seqs_.size() - free_ids_.size()); }

  int blocks_needed(int sid, int new_tokens) const {
    const Seq& s = at(sid);
    int need = (s.length + new_tokens + bs_ - 1) / bs_ - static_cast<int>(s.blocks.size());
    if (new_tokens > 0 && s.length % bs_ != 0 && !s.blocks.empty() &&
        refcount_[static_cast<size_t>(s.blocks[static_cast<size_t>(s.length / bs_)])] > 1)
      ++need;
    return std::max(0, need);
  }

  // A token that was fed from the device before the host had read it: fill it in once it is known.
  bool patch(int sid, int index, int token) {
    if (!live(sid)) return false;
    Seq& s = seqs_[static_cast<size_t>(sid)];
    if (index < 0 || static_cast<size_t>(index) >= s.tokens.size() || s.tokens[static_cast<size_t>(index)] != -1) return false;
    s.tokens[static_cast<size_t>(index)] = token;
    return true;
  }

  // One step: chunk i appends counts[i] tokens (taken in order from `flat`) to sequence seqs[i], wants logits for its
  // last logits[i] rows, and output[i] tells whether its tokens are model output.
  py::dict plan(const std::vector<int>& seqs, const std::vector<int>& counts, const std::vector<int32_t>& flat,
                const std::vector<int>& logits, const std::vector<int>& output, bool device_tokens, int max_tokens) {
    if (seqs.size() != counts.size() || seqs.size() != logits.size() || seqs.size() != output.size())
      throw std::invalid_argument("plan: chunk arrays differ in length");
    // pass 0: everything that can fail is checked before any state changes, so a refused step leaves the sequences,
    // the block pool and the previous plan exactly as they were
    {
      std::vector<int> grown(seqs_.size(), 0), new_blocks(seqs_.size(), 0);
      std::vector<std::pair<int32_t, int>> released;               // shared blocks this step stops sharing, with counts
      size_t have = 0;
      long total = 0, need_blocks = 0;
      for (size_t i = 0; i < seqs.size(); ++i) {
        const int n = counts[i];
        if (n < 0) throw std::invalid_argument("plan: negative token count");
        if (n == 0) continue;
        if (device_tokens && n != 1) throw std::invalid_argument("device_tokens needs one-token chunks");
        have += static_cast<size_t>(n);
        if (have > flat.size()) throw std::invalid_argument("plan: fewer tokens than the counts say");
        const int sid = seqs[i];
        const Seq& s = at(sid);
        const size_t si = static_cast<size_t>(sid);
        const int len = s.length + grown[si];
        if (len + n > ctx_)
          throw std::invalid_argument("sequence " + std::to_string(sid) + " would exceed the context length " + std::to_string(ctx_));
        total += n;
        if (total > max_tokens)
          throw std::invalid_argument(std::to_string(total) + " tokens exceed max_tokens " + std::to_string(max_tokens));
        long need = (len + n + bs_ - 1) / bs_ - static_cast<long>(s.blocks.size()) - new_blocks[si];
        if (need < 0) need = 0;
        if (grown[si] == 0 && s.length % bs_ != 0) {
          const int32_t last = s.blocks[static_cast<size_t>(s.length / bs_)];
          int refs = refcount_[static_cast<size_t>(last)];
          auto it = std::find_if(released.begin(), released.end(), [&](const auto& p) { return p.first == last; });
          if (it != released.end()) refs -= it->second;          // earlier chunks of this step already copied away
          if (refs > 1) {                                        // copy-on-write of the shared partial block
            ++need_blocks;
            if (it != released.end()) ++it->second; else released.emplace_back(last, 1);
          }
        }
        new_blocks[si] += static_cast<int>(need);
        need_blocks += need;
        grown[si] += n;
      }
      if (need_blocks > static_cast<long>(free_blocks_.size())) throw std::runtime_error("KV cache exhausted");
    }
    tok_.clear(); pos_.clear(); slot_.clear(); rseq_.clear(); logit_rows_.clear();
    std::vector<int> out_rows, logit_seq, table_changed;
    std::vector<std::pair<int, int>> cows, patches;
    py::list runs;
    int run_kind = -1, run_r0 = 0, run_r1 = 0, run_seq = -1;     // pending "paged" run being extended
    auto flush_run = [&] {
      if (run_kind >= 0) runs.append(py::make_tuple(run_kind == 0 ? "flash" : "paged", run_r0, run_r1, run_seq));
      run_kind = -1;
    };
    long prefill = 0, decode = 0;
    size_t cursor = 0;
    for (size_t i = 0; i < seqs.size(); ++i) {
      const int n = counts[i];
      if (n < 0) throw std::invalid_argument("plan: negative token count");
      if (n == 0) continue;
      if (device_tokens && n != 1) throw std::invalid_argument("device_tokens needs one-token chunks");
      if (cursor + static_cast<size_t>(n) > flat.size()) throw std::invalid_argument("plan: fewer tokens than the counts say");
      const int sid = seqs[i];
      Seq& s = at(sid);
      if (s.length + n > ctx_)
        throw std::invalid_argument("sequence " + std::to_string(sid) + " would exceed the context length " + std::to_string(ctx_));
      if (static_cast<long>(tok_.size()) + n > max_tokens)
        throw std::invalid_argument(std::to_string(tok_.size() + static_cast<size_t>(n)) + " tokens exceed max_tokens " +
                                    std::to_string(max_tokens));
      // make positions [length, length + n) writable
      bool changed = false;
      if (s.length % bs_ != 0) {
        int32_t& last = s.blocks[static_cast<size_t>(s.length / bs_)];
        if (refcount_[static_cast<size_t>(last)] > 1) {        // shared partial block: copy before writing
          const int32_t nb = take();
          cows.emplace_back(last, nb);
          release(last);
          last = nb;
          changed = true;
        }
      }
      while (static_cast<int>(s.blocks.size()) * bs_ < s.length + n) {
        s.blocks.push_back(take());
        changed = true;
      }
      if (changed) table_changed.push_back(sid);
      const int r0 = static_cast<int>(tok_.size());
      const bool fresh = s.length == 0 && n > 1;
      for (int j = 0; j < n; ++j) {
        const int p = s.length + j;
        tok_.push_back(device_tokens ? 0 : flat[cursor + static_cast<size_t>(j)]);
        pos_.push_back(p);
        slot_.push_back(s.blocks[static_cast<size_t>(p / bs_)] * bs_ + p % bs_);
        rseq_.push_back(sid);
        if (output[i]) out_rows.push_back(r0 + j);
      }
      if (fresh) {
        flush_run();
        runs.append(py::make_tuple("flash", r0, r0 + n, sid));
        prefill += n;
      } else {
        if (run_kind == 1 && run_r1 == r0) {
          run_r1 = r0 + n;
        } else {
          flush_run();
          run_kind = 1; run_r0 = r0; run_r1 = r0 + n; run_seq = -1;
        }
        if (s.length == 0 || n > 1) prefill += n; else decode += n;
      }
      const int k = std::min(logits[i], n);
      for (int j = n - k; j < n; ++j) {
        logit_rows_.push_back(r0 + j);
        logit_seq.push_back(sid);
      }
      if (!output[i] && s.length == s.n_prompt) s.n_prompt += n;
      if (device_tokens) {
        patches.emplace_back(sid, static_cast<int>(s.tokens.size()));
        s.tokens.push_back(-1);
      } else {
        s.tokens.insert(s.tokens.end(), flat.begin() + static_cast<long>(cursor), flat.begin() + static_cast<long>(cursor) + n);
      }
      s.length += n;
      cursor += static_cast<size_t>(n);
    }
    flush_run();
    py::dict out;
    out["tokens"] = static_cast<int>(tok_.size());
    out["logit_rows"] = static_cast<int>(logit_rows_.size());
    out["prefill_tokens"] = prefill;
    out["decode_tokens"] = decode;
    out["runs"] = runs;
    out["out_rows"] = out_rows;
    out["logit_seq"] = logit_seq;
    out["cows"] = cows;
    out["tables"] = table_changed;
    out["patches"] = patches;
    return out;
  }

  // Fills the staging rows [6, width] (int32, row-major) from the last plan; columns past the batch are padding.
  void write(uintptr_t ptr, int width) const {
    const int n = static_cast<int>(tok_.size()), r = static_cast<int>(logit_rows_.size());
    if (ptr == 0 || width < n || width < r) throw std::invalid_argument("write: staging buffer is too small");
    int32_t* h = reinterpret_cast<int32_t*>(ptr);
    const size_t w = static_cast<size_t>(width);
    for (int i = 0; i < width; ++i) {
      const bool in = i < n;
      const size_t c = static_cast<size_t>(i);
      h[0 * w + c] = in ? tok_[c] : 0;
      h[1 * w + c] = in ? pos_[c] : 0;
      h[2 * w + c] = in ? slot_[c] : -1;
      h[3 * w + c] = in ? rseq_[c] : 0;
      h[4 * w + c] = in ? pos_[c] + 1 : 0;
      h[5 * w + c] = i < r ? logit_rows_[c] : 0;
    }
  }

 private:
  Seq& at(int sid) {
    if (!live(sid)) throw py::key_error("unknown sequence " + std::to_string(sid));
    return seqs_[static_cast<size_t>(sid)];
  }
  const Seq& at(int sid) const {
    if (!live(sid)) throw py::key_error("unknown sequence " + std::to_string(sid));
    return seqs_[static_cast<size_t>(sid)];
  }
  void release(int32_t b) {
    if (--refcount_[static_cast<size_t>(b)] == 0) free_blocks_.push_back(b);
  }
  int32_t take() {
    if (free_blocks_.empty()) throw std::runtime_error("KV cache exhausted");
    const int32_t b = free_blocks_.back();
    free_blocks_.pop_back();
    refcount_[static_cast<size_t>(b)] = 1;
    return b;
  }

  int bs_, ctx_;
  std::vector<int> refcount_;
  std::vector<int32_t> free_blocks_;
  std::vector<int> free_ids_;
  std::vector<Seq> seqs_;
  std::vector<int32_t> tok_, pos_, slot_, rseq_, logit_rows_;
};

}  // namespace

void bind_kv_sched(py::module_& m) {
  py::class_<KvScheduler>(m, "KvScheduler")
      .def(py::init<int, int, int, int>(), py::arg("n_blocks"), py::arg("block_size"), py::arg("max_seqs"), py::arg("ctx"))
      .def("add", &KvScheduler::add)
      .def("fork", &KvScheduler::fork)
      .def("free", &KvScheduler::free)
      .def("truncate", &KvScheduler::truncate)
      .def("live", &KvScheduler::live)
      .def("length", &KvScheduler::length)
      .def("n_prompt", &KvScheduler::n_prompt)
      .def("tokens", &KvScheduler::tokens)
      .def("blocks", &KvScheduler::blocks)
      .def("refcount", &KvScheduler::refcount)
      .def("free_blocks", &KvScheduler::free_blocks)
      .def("total_blocks", &KvScheduler::total_blocks)
      .def("live_sequences", &KvScheduler::live_sequences)
      .def("blocks_needed", &KvScheduler::blocks_needed)
      .def("patch", &KvScheduler::patch)
      .def("plan", &KvScheduler::plan, py::arg("seqs"), py::arg("counts"), py::arg("flat"), py::arg("logits"), py::arg("output"),
           py::arg("device_tokens"), py::arg("max_tokens"))
      .def("write", &KvScheduler::write);
}
