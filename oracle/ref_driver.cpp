// Test infrastructure, not product code.
//
// Drives the UNMODIFIED litnicelm reference (linked from its own sources by
// oracle/Makefile) on explicit token-id vectors. The reference's `infer` and
// `inspect` commands only accept text prompts, and their runtime object lives
// in an anonymous namespace (src/model/inference.cpp:27,49-71), so this
// program repeats that object's set-up steps around the reference's own
// Transformer::forward, and restates the file-local token selectors and loop
// guard (src/model/inference.cpp:188-296).
//
// The backend is whatever `backend.library` in the YAML names: the reference
// CPU plugin (oracle), or the B200 plugin (drop-in check: the reference's model
// code then runs on the plugin through the C ABI with no change).
//
// Usage:
//   ref_driver --config cfg.yaml --vocab V --ids ids.i32 --mode forward --out logits.f32
//   ref_driver --config cfg.yaml --vocab V --ids ids.i32 --mode generate
//              --max-new N --temp T --top-k K --top-p P --seed S
//              --out tokens.i32 [--logits-out lastrow_logits.f32] [--times-out t.f64]
//   forward : writes all s rows of logits, s*V floats.
//   generate: writes the generated ids (int32), optionally the last-row logits
//             of every step (steps*V floats) and per-step wall seconds (f64).

#include "algo/transformer.hpp"
#include "backend/device_backend.hpp"
#include "checkpoint.hpp"
#include "host_tensor_stage.hpp"
#include "memory/inference_memory_manager.hpp"
#include "ops.hpp"
#include <config.hpp>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct Args {
  std::string config, ids, mode = "forward", out, logits_out, times_out;
  uint32_t vocab = 0, max_new = 0, top_k = 0, seed = 12345;
  float temp = 0.0f, top_p = 1.0f;
};

Args parse(int argc, char **argv) {
  Args a;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--config") a.config = v;
    else if (k == "--ids") a.ids = v;
    else if (k == "--mode") a.mode = v;
    else if (k == "--out") a.out = v;
    else if (k == "--logits-out") a.logits_out = v;
    else if (k == "--times-out") a.times_out = v;
    else if (k == "--vocab") a.vocab = static_cast<uint32_t>(std::stoul(v));
    else if (k == "--max-new") a.max_new = static_cast<uint32_t>(std::stoul(v));
    else if (k == "--top-k") a.top_k = static_cast<uint32_t>(std::stoul(v));
    else if (k == "--seed") a.seed = static_cast<uint32_t>(std::stoul(v));
    else if (k == "--temp") a.temp = std::stof(v);
    else if (k == "--top-p") a.top_p = std::stof(v);
    else throw std::runtime_error("ref_driver: unknown flag " + k);
  }
  if (a.config.empty() || a.ids.empty() || a.out.empty() || a.vocab == 0)
    throw std::runtime_error("ref_driver: --config --vocab --ids --out are required");
  return a;
}

template <class T> std::vector<T> read_all(const std::string &path) {
  std::ifstream in(path, std::ios::binary | std::ios::ate);
  if (!in) throw std::runtime_error("ref_driver: cannot open " + path);
  const std::streamsize n = in.tellg();
  in.seekg(0);
  std::vector<T> v(static_cast<size_t>(n) / sizeof(T));
  in.read(reinterpret_cast<char *>(v.data()), n);
  return v;
}

template <class T> void write_all(const std::string &path, const std::vector<T> &v) {
  std::ofstream out(path, std::ios::binary);
  out.write(reinterpret_cast<const char *>(v.data()),
            static_cast<std::streamsize>(v.size() * sizeof(T)));
  if (!out) throw std::runtime_error("ref_driver: cannot write " + path);
}

// First index of the maximum, strict '>' (inference.cpp:188-198).
int32_t pick_greedy(const std::vector<float> &row) {
  int32_t best = 0;
  float bestv = row.at(0);
  for (size_t i = 1; i < row.size(); ++i)
    if (row[i] > bestv) { bestv = row[i]; best = static_cast<int32_t>(i); }
  return best;
}

// Temperature / top-k / top-p draw (inference.cpp:200-263): descending sort on
// double(logit)/temp, top-k truncation, shortest prefix whose cumulative
// probability reaches top_p, then one std::discrete_distribution draw.
int32_t pick_sampled(const std::vector<float> &row, float temp, uint32_t top_k,
                     float top_p, std::mt19937 &rng) {
  if (temp <= 0.0f || top_k == 1) return pick_greedy(row);
  if (!(top_p > 0.0f && top_p <= 1.0f))
    throw std::runtime_error("top_p must be in (0,1]");
  struct Cand { int32_t id; double x; };
  std::vector<Cand> c;
  c.reserve(row.size());
  const double inv_temp = 1.0 / static_cast<double>(temp);
  for (size_t i = 0; i < row.size(); ++i)
    c.push_back(Cand{static_cast<int32_t>(i), static_cast<double>(row[i]) * inv_temp});
  std::sort(c.begin(), c.end(), [](const Cand &a, const Cand &b) { return a.x > b.x; });
  if (top_k > 0 && top_k < c.size()) c.resize(top_k);
  if (top_p < 1.0f) {
    const double mx = c.front().x;
    std::vector<double> p(c.size());
    double sum = 0.0;
    for (size_t i = 0; i < c.size(); ++i) { p[i] = std::exp(c[i].x - mx); sum += p[i]; }
    double cum = 0.0;
    size_t keep = 0;
    for (; keep < c.size(); ++keep) {
      cum += p[keep] / sum;
      if (cum >= static_cast<double>(top_p)) { ++keep; break; }
    }
    c.resize(std::max<size_t>(1, keep));
  }
  const double mx = c.front().x;
  std::vector<double> w(c.size());
  for (size_t i = 0; i < c.size(); ++i) w[i] = std::exp(c[i].x - mx);
  std::discrete_distribution<size_t> dist(w.begin(), w.end());
  return c[dist(rng)].id;
}

struct Runtime {
  Config cfg;
  std::unique_ptr<DeviceBackend> backend;
  std::unique_ptr<InferenceMemoryManager> mm;
  std::unique_ptr<Ops> ops;
  std::unique_ptr<Transformer> model;

  Runtime(const std::string &config_path, uint32_t vocab) {
    cfg = Config::load_from_file(config_path);
    cfg.model.target_vocab_size = vocab;
    backend = DeviceBackend::create_instance(cfg);
    mm = std::make_unique<InferenceMemoryManager>(cfg, *backend);
    ops = std::make_unique<Ops>(*backend);
    model = std::make_unique<Transformer>(cfg, mm->tensor_store(), nullptr, *ops, nullptr);
    uint64_t step = 0;
    uint32_t epoch = 0;
    std::string err;
    if (!load_checkpoint(cfg.paths.model_file_best, cfg.model, cfg.conf_version,
                         cfg.memory.alignment_bytes, *backend, mm->data_arena(),
                         mm->adam_state(), step, epoch, nullptr, &err))
      throw std::runtime_error("ref_driver: checkpoint load failed: " + err);
  }

  // Same steps as forward_prompt + stage_to_cpu (inference.cpp:93-143).
  Tensor forward(const std::vector<int32_t> &ids) {
    const int64_t s = static_cast<int64_t>(ids.size());
    TensorView ids_t = mm->tensor_store().temp_infer_ids(s);
    Tensor ids_host = Tensor::make_cpu(DType::I32, ids_t.shape());
    std::memcpy(ids_host.view().data(), ids.data(), ids.size() * sizeof(int32_t));
    host_tensor_stage::copy_from_cpu(*backend, ids_host.view(), ids_t, "ref_driver(ids)");
    TensorView logits = mm->tensor_store().temp_infer_logits(s);
    model->forward(ids_t, logits);
    return host_tensor_stage::stage_to_cpu(*backend, logits, "ref_driver(logits)");
  }
};

std::vector<float> last_row(const Tensor &logits_host, int64_t vocab) {
  TensorView v = logits_host.view();
  if (v.rank() == 3) v = v.select(0, 0);
  const int64_t r = v.dim(0) - 1;
  std::vector<float> row(static_cast<size_t>(vocab));
  for (int64_t c = 0; c < vocab; ++c) row[static_cast<size_t>(c)] = v.at_f32(r, c);
  return row;
}

int run(const Args &a) {
  Runtime rt(a.config, a.vocab);
  std::vector<int32_t> ids = read_all<int32_t>(a.ids);
  if (ids.empty()) ids.push_back(0);  // inference.cpp:121-123
  const int64_t V = a.vocab;

  if (a.mode == "forward") {
    const auto t0 = std::chrono::steady_clock::now();
    Tensor lh = rt.forward(ids);
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    TensorView v = lh.view().select(0, 0);
    std::vector<float> all(static_cast<size_t>(v.dim(0) * V));
    for (int64_t r = 0; r < v.dim(0); ++r)
      for (int64_t c = 0; c < V; ++c) all[static_cast<size_t>(r * V + c)] = v.at_f32(r, c);
    write_all(a.out, all);
    std::printf("{\"mode\":\"forward\",\"rows\":%lld,\"seconds\":%.6f}\n",
                static_cast<long long>(v.dim(0)), dt);
    return 0;
  }
  if (a.mode != "generate") throw std::runtime_error("ref_driver: bad --mode");

  std::mt19937 rng(a.seed);
  const uint32_t max_seq = rt.cfg.model.max_seq_len;
  std::vector<int32_t> generated;
  std::vector<float> step_logits;
  std::vector<double> times;
  // Loop guard of generate_text (inference.cpp:278).
  for (uint32_t step = 0; step < a.max_new && ids.size() < max_seq; ++step) {
    const auto t0 = std::chrono::steady_clock::now();
    Tensor lh = rt.forward(ids);
    const std::vector<float> row = last_row(lh, V);
    const int32_t next = pick_sampled(row, a.temp, a.top_k, a.top_p, rng);
    times.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    ids.push_back(next);
    generated.push_back(next);
    if (!a.logits_out.empty()) step_logits.insert(step_logits.end(), row.begin(), row.end());
  }
  write_all(a.out, generated);
  if (!a.logits_out.empty()) write_all(a.logits_out, step_logits);
  if (!a.times_out.empty()) write_all(a.times_out, times);
  double total = 0.0;
  for (double t : times) total += t;
  std::printf("{\"mode\":\"generate\",\"tokens\":%zu,\"seconds\":%.6f}\n", generated.size(), total);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  try {
    return run(parse(argc, argv));
  } catch (const std::exception &e) {
    std::fprintf(stderr, "ref_driver: %s\n", e.what());
    return 1;
  }
}
