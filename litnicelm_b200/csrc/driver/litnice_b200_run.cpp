// litnice_b200_run: host driver of the native token loop.
//
// Reads the same YAML keys as `litnicelm infer` / `inspect`
// (litnicelm src/config/config_mapper.cpp:124-189), loads the plugin named by
// backend.library with dlopen, loads paths.model_file_best, and prints the same
// [INFERENCE] lines as generate_text (src/model/inference.cpp:265-296,
// include/report_interface.hpp:94-97), but the loop itself runs on the GPU
// through the litnice_b200_* entry points: no logits return per token.
//
//   litnice_b200_run infer   --config cfg.yaml [--prompt TEXT | --ids-file ids.i32]
//                            [--max_new N] [--temp T] [--top_k K] [--top_p P] [--seed S]
//                            [--streams N] [--gpus G] [--out-ids-file out.i32]
//   litnice_b200_run inspect --config cfg.yaml [--prompt TEXT | --ids-file ids.i32]
//   litnice_b200_run partition --streams N --gpus G      (prints the split; needs no GPU)
//
// --ids-file holds int32 token ids, streams*len of them (row-major); with
// --streams N the N rows are decoded in lockstep with seeds seed, seed+1, ...
// With --gpus G the streams are cut into G contiguous blocks, one host thread
// per GPU decodes its block on its own session (weights replicated, nothing is
// exchanged between GPUs), and the threads are joined before anything is printed.
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <map>
#include <sstream>
#include <chrono>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../../../include/litnice_backend_b200.h"

namespace {

std::string trim(const std::string &s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace((unsigned char)s[a])) ++a;
  while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}

std::string unquote(std::string v) {
  if (v.size() >= 2 && ((v.front() == '"' && v.back() == '"') || (v.front() == '\'' && v.back() == '\'')))
    v = v.substr(1, v.size() - 2);
  std::string out;
  for (size_t i = 0; i < v.size(); ++i) {
    if (v[i] == '\\' && i + 1 < v.size()) {
      const char n = v[++i];
      out += n == 'n' ? '\n' : n == 't' ? '\t' : n == 'r' ? '\r' : n;
    } else {
      out += v[i];
    }
  }
  return out;
}

// Flat YAML as the reference reads it (src/utils/yaml_parser.cpp:9-76): nesting
// by indentation, '#' starts a comment, values optionally quoted.
std::map<std::string, std::string> parse_yaml(const std::string &path) {
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open config " + path);
  std::map<std::string, std::string> out;
  std::vector<std::pair<int, std::string>> stack;
  std::string line;
  while (std::getline(in, line)) {
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line = line.substr(0, hash);
    if (trim(line).empty()) continue;
    int indent = 0;
    while (indent < (int)line.size() && line[indent] == ' ') ++indent;
    const std::string body = trim(line);
    const size_t colon = body.find(':');
    if (colon == std::string::npos) continue;
    const std::string key = trim(body.substr(0, colon)), val = trim(body.substr(colon + 1));
    while (!stack.empty() && stack.back().first >= indent) stack.pop_back();
    std::string full;
    for (auto &p : stack) full += p.second + ".";
    full += key;
    if (val.empty()) stack.emplace_back(indent, key);
    else out[full] = unquote(val);
  }
  return out;
}

struct Tokenizer {
  std::string type;
  int vocab = 0;
  std::vector<std::string> seen;  // only_seen_chars: id -> character

  // character: byte value is the id (include/tokenizer.hpp, character tokenizer);
  // only_seen_chars: position in char_seen.json's "vocab" list
  // (only_seen_chars_tokenizer_plugin.cpp:249-262).
  std::vector<int32_t> encode(const std::string &text) const {
    std::vector<int32_t> ids;
    for (unsigned char c : text) {
      if (seen.empty()) {
        if ((int)c >= vocab) throw std::runtime_error("prompt byte outside the character vocabulary");
        ids.push_back((int32_t)c);
      } else {
        const std::string ch(1, (char)c);
        auto it = std::find(seen.begin(), seen.end(), ch);
        if (it == seen.end()) throw std::runtime_error("prompt character not in char_seen.json");
        ids.push_back((int32_t)(it - seen.begin()));
      }
    }
    return ids;
  }
  std::string decode(int32_t id) const {
    if (id < 0 || id >= vocab) return "<invalid>";
    if (seen.empty()) return std::string(1, (char)id);
    return seen[(size_t)id];
  }
};

Tokenizer make_tokenizer(const std::map<std::string, std::string> &cfg) {
  Tokenizer t;
  t.type = cfg.at("tokenizer.type");
  t.vocab = std::stoi(cfg.at("tokenizer.target_vocab_size"));
  if (t.type == "only_seen_chars" || t.type == "char_seen" || t.type == "seen_chars") {
    const std::string path = cfg.at("tokenizer.artifacts_dir") + "/char_seen.json";
    std::ifstream in(path);
    if (!in) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << in.rdbuf();
    const std::string js = ss.str();
    size_t p = js.find("\"vocab\"");
    if (p == std::string::npos) throw std::runtime_error("char_seen.json has no vocab list");
    p = js.find('[', p);
    const size_t end = js.find(']', p);
    while (true) {
      const size_t q0 = js.find('"', p);
      if (q0 == std::string::npos || q0 > end) break;
      size_t q1 = q0 + 1;
      std::string item;
      while (q1 < js.size() && js[q1] != '"') {
        if (js[q1] == '\\' && q1 + 1 < js.size()) {
          const char n = js[++q1];
          item += n == 'n' ? '\n' : n == 't' ? '\t' : n == 'r' ? '\r' : n;
        } else {
          item += js[q1];
        }
        ++q1;
      }
      t.seen.push_back(item);
      p = q1 + 1;
    }
    t.vocab = (int)t.seen.size();
  } else if (!(t.type == "character" || t.type == "char" || t.type == "bytes")) {
    throw std::runtime_error("litnice_b200_run supports tokenizer.type character and only_seen_chars");
  }
  return t;
}

std::string escape_for_log(const std::string &tok) {  // inference.cpp:153-186
  std::string out;
  for (char ch : tok) {
    switch (ch) {
      case '\\': out += "\\\\"; break;
      case '"': out += "\\\""; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default: out += ch;
    }
  }
  return out;
}

void report(const char *event, uint32_t step, float value, const std::string &msg) {
  std::cout << "[INFERENCE][" << event << "] step=" << step << " val=" << std::to_string(value) << " " << msg
            << "\n";
}

// Contiguous blocks; the first total % parts blocks carry one stream more.
void partition_streams(int total, int parts, int index, int *first, int *count) {
  const int base = total / parts, extra = total % parts;
  *count = base + (index < extra ? 1 : 0);
  *first = index * base + std::min(index, extra);
}

struct Api {
  void *handle = nullptr;
  decltype(&litnice_b200_session_create) create = nullptr;
  decltype(&litnice_b200_session_create_on) create_on = nullptr;
  decltype(&litnice_b200_session_destroy) destroy = nullptr;
  decltype(&litnice_b200_last_error) last_error = nullptr;
  decltype(&litnice_b200_load_checkpoint) load_checkpoint = nullptr;
  decltype(&litnice_b200_generate) generate = nullptr;
  decltype(&litnice_b200_inspect) inspect = nullptr;
  decltype(&litnice_b200_forward) forward = nullptr;
  decltype(&litnice_b200_get_stats) get_stats = nullptr;

  explicit Api(const std::string &path) {
    handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!handle) throw std::runtime_error(std::string("cannot load ") + path + ": " + dlerror());
#define RESOLVE(field, sym)                                        \
  field = reinterpret_cast<decltype(field)>(dlsym(handle, sym));   \
  if (!field) throw std::runtime_error(std::string("missing symbol ") + sym)
    RESOLVE(create, "litnice_b200_session_create");
    RESOLVE(create_on, "litnice_b200_session_create_on");
    RESOLVE(destroy, "litnice_b200_session_destroy");
    RESOLVE(last_error, "litnice_b200_last_error");
    RESOLVE(load_checkpoint, "litnice_b200_load_checkpoint");
    RESOLVE(generate, "litnice_b200_generate");
    RESOLVE(inspect, "litnice_b200_inspect");
    RESOLVE(forward, "litnice_b200_forward");
    RESOLVE(get_stats, "litnice_b200_get_stats");
#undef RESOLVE
  }
};

int run(int argc, char **argv) {
  if (argc < 2) throw std::runtime_error("usage: litnice_b200_run infer|inspect --config cfg.yaml [...]");
  const std::string mode = argv[1];
  std::map<std::string, std::string> opt;
  for (int i = 2; i + 1 < argc; i += 2) opt[argv[i]] = argv[i + 1];
  if (mode == "partition") {
    const int total = std::stoi(opt.at("--streams")), parts = std::stoi(opt.at("--gpus"));
    if (total < 0 || parts <= 0) throw std::runtime_error("partition needs --streams >= 0 and --gpus >= 1");
    for (int g = 0; g < parts; ++g) {
      int first = 0, count = 0;
      partition_streams(total, parts, g, &first, &count);
      std::cout << "gpu " << g << " first " << first << " count " << count << "\n";
    }
    return 0;
  }
  if (!opt.count("--config")) throw std::runtime_error("--config is required");
  auto cfg = parse_yaml(opt["--config"]);
  auto get = [&](const char *flag, const char *key) { return opt.count(flag) ? opt[flag] : cfg.at(key); };

  Tokenizer tok = make_tokenizer(cfg);
  litnice_b200_dims d{};
  d.n_layers = std::stoi(cfg.at("model.n_layers"));
  d.n_heads = std::stoi(cfg.at("model.n_heads"));
  d.d_model = std::stoi(cfg.at("model.d_model"));
  d.d_ff = std::stoi(cfg.at("model.d_ff"));
  d.max_seq_len = std::stoi(cfg.at("model.max_seq_len"));
  d.vocab_size = tok.vocab;  // model.target_vocab_size follows the tokenizer (inference.cpp:64-65)
  d.alignment_bytes = std::stoull(cfg.at("memory.alignment_bytes"));

  const std::string prompt = get("--prompt", "inference.prompt");
  const int max_new = std::stoi(get("--max_new", "inference.max_new"));
  litnice_b200_sampling sp{std::stof(get("--temp", "inference.temp")),
                           (uint32_t)std::stoul(get("--top_k", "inference.top_k")),
                           std::stof(get("--top_p", "inference.top_p"))};
  const uint32_t seed = (uint32_t)std::stoul(get("--seed", "inference.seed"));
  const int streams = opt.count("--streams") ? std::stoi(opt["--streams"]) : 1;
  const int gpus = opt.count("--gpus") ? std::stoi(opt["--gpus"]) : 1;
  if (streams <= 0 || gpus <= 0) throw std::runtime_error("--streams and --gpus must be positive");

  std::vector<int32_t> ids;
  if (opt.count("--ids-file")) {
    std::ifstream in(opt["--ids-file"], std::ios::binary | std::ios::ate);
    if (!in) throw std::runtime_error("cannot open --ids-file");
    const std::streamsize n = in.tellg();
    in.seekg(0);
    ids.resize((size_t)n / 4);
    in.read(reinterpret_cast<char *>(ids.data()), n);
  } else {
    ids = tok.encode(prompt);
    if (ids.empty()) ids.push_back(0);  // inference.cpp:121-123
    std::vector<int32_t> one = ids;
    for (int i = 1; i < streams; ++i) ids.insert(ids.end(), one.begin(), one.end());
  }
  if (ids.size() % (size_t)streams != 0) throw std::runtime_error("ids do not divide into --streams rows");
  const int len = (int)(ids.size() / (size_t)streams);

  Api api(cfg.at("backend.library"));
  std::cout << "[DeviceBackend] Loaded backend library: " << cfg.at("backend.library") << " (native loop)\n";
  const std::string ckpt = cfg.at("paths.model_file_best");

  if (mode == "infer" && gpus > 1) {
    // One host thread per GPU, each with its own session and its own block of streams.
    std::vector<uint32_t> seeds((size_t)streams);
    for (int i = 0; i < streams; ++i) seeds[(size_t)i] = seed + (uint32_t)i;
    std::vector<int32_t> out((size_t)streams * (size_t)std::max(1, max_new));
    std::vector<int> counts((size_t)gpus, 0);
    std::vector<std::string> errors((size_t)gpus);
    std::vector<double> device_ms((size_t)gpus, 0.0);
    const auto t0 = std::chrono::steady_clock::now();
    std::vector<std::thread> workers;
    for (int g = 0; g < gpus; ++g) {
      workers.emplace_back([&, g]() {
        int first = 0, n = 0;
        partition_streams(streams, gpus, g, &first, &n);
        if (n == 0) return;
        litnice_b200_session *ws = nullptr;
        auto fail = [&](const char *what, int code) {
          errors[(size_t)g] = std::string(what) + " failed on GPU " + std::to_string(g) + " (" + std::to_string(code) +
                              "): " + api.last_error(ws);
          if (ws) api.destroy(ws);
        };
        int rc = api.create_on(&d, n, g, &ws);
        if (rc != LITNICE_B200_OK) return fail("session_create", rc);
        rc = api.load_checkpoint(ws, ckpt.c_str());
        if (rc != LITNICE_B200_OK) return fail("load_checkpoint", rc);
        rc = api.generate(ws, ids.data() + (size_t)first * len, n, len, max_new, &sp, seeds.data() + first,
                          out.data() + (size_t)first * std::max(1, max_new), &counts[(size_t)g]);
        if (rc != LITNICE_B200_OK) return fail("generate", rc);
        litnice_b200_stats stt{};
        api.get_stats(ws, &stt);
        device_ms[(size_t)g] = stt.device_ms;
        api.destroy(ws);
      });
    }
    for (auto &w : workers) w.join();
    const double wall_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    for (auto &e : errors)
      if (!e.empty()) throw std::runtime_error(e);
    const int count = counts[0];
    report("START", 0, 0.0f, "Inference started: " + std::to_string(streams) + " streams on " + std::to_string(gpus) +
                                 " GPUs, max_new=" + std::to_string(max_new));
    for (int b = 0; b < streams; ++b) {
      std::string text;
      for (int i = 0; i < len; ++i) text += tok.decode(ids[(size_t)b * len + i]);
      for (int i = 0; i < count; ++i) text += tok.decode(out[(size_t)b * max_new + i]);
      if (b == 0) report("END", (uint32_t)(len + count), 0.0f, "Inference complete");
      report("TOKEN_GEN", 0, 0.0f, text);
    }
    if (opt.count("--out-ids-file")) {
      std::ofstream o(opt["--out-ids-file"], std::ios::binary);
      for (int b = 0; b < streams; ++b)
        o.write(reinterpret_cast<const char *>(out.data() + (size_t)b * max_new), (std::streamsize)count * 4);
    }
    const double slowest = *std::max_element(device_ms.begin(), device_ms.end());
    std::fprintf(stderr,
                 "[litnice_b200] %d streams x %d tokens on %d GPUs: slowest GPU %.3f ms on device (%.1f tokens/s), "
                 "%.1f ms wall including weight loading\n",
                 streams, count, gpus, slowest, slowest > 0 ? (double)streams * count * 1e3 / slowest : 0.0, wall_ms);
    return 0;
  }

  litnice_b200_session *s = nullptr;
  int rc = api.create(&d, streams, &s);
  auto check = [&](int code, const char *what) {
    if (code != LITNICE_B200_OK) {
      const std::string msg = std::string(what) + " failed (" + std::to_string(code) + "): " + api.last_error(s);
      if (s) api.destroy(s);
      throw std::runtime_error(msg);
    }
  };
  check(rc, "session_create");
  check(api.load_checkpoint(s, ckpt.c_str()), "load_checkpoint");

  if (mode == "infer") {
    std::ostringstream start;
    start << "Inference started: prompt=\"" << escape_for_log(prompt) << "\" max_new=" << max_new
          << " temp=" << sp.temp << " top_k=" << sp.top_k << " top_p=" << sp.top_p << " seed=" << seed;
    report("START", 0, 0.0f, start.str());
    std::vector<uint32_t> seeds((size_t)streams);
    for (int i = 0; i < streams; ++i) seeds[(size_t)i] = seed + (uint32_t)i;
    std::vector<int32_t> out((size_t)streams * (size_t)std::max(1, max_new));
    int count = 0;
    check(api.generate(s, ids.data(), streams, len, max_new, &sp, seeds.data(), out.data(), &count), "generate");
    for (int b = 0; b < streams; ++b) {
      std::string text;
      for (int i = 0; i < len; ++i) text += tok.decode(ids[(size_t)b * len + i]);
      for (int i = 0; i < count; ++i) {
        const int32_t t = out[(size_t)b * max_new + i];
        if (streams == 1)
          report("TOKEN_GEN", (uint32_t)i + 1, (float)t,
                 "Generated token id=" + std::to_string(t) + " token=\"" + escape_for_log(tok.decode(t)) + "\"");
        text += tok.decode(t);
      }
      if (b == 0) report("END", (uint32_t)(len + count), 0.0f, "Inference complete");
      report("TOKEN_GEN", 0, 0.0f, text);
    }
    if (opt.count("--out-ids-file")) {
      std::ofstream o(opt["--out-ids-file"], std::ios::binary);
      for (int b = 0; b < streams; ++b)
        o.write(reinterpret_cast<const char *>(out.data() + (size_t)b * max_new), (std::streamsize)count * 4);
    }
    litnice_b200_stats stt{};
    api.get_stats(s, &stt);
    std::fprintf(stderr, "[litnice_b200] %lld tokens in %.3f ms on device (%.1f tokens/s), %lld kernel launches\n",
                 (long long)stt.tokens, stt.device_ms, stt.device_ms > 0 ? stt.tokens * 1e3 / stt.device_ms : 0.0,
                 (long long)stt.kernel_launches);
  } else if (mode == "inspect") {
    // inspect_distribution (inference.cpp:298-359) for stream 0
    std::vector<float> logits((size_t)streams * d.vocab_size), probs((size_t)streams * d.vocab_size);
    check(api.forward(s, ids.data(), streams, len, 0, logits.data()), "forward");
    check(api.inspect(s, ids.data(), streams, len, probs.data()), "inspect");
    std::vector<int32_t> order((size_t)d.vocab_size);
    for (int i = 0; i < d.vocab_size; ++i) order[(size_t)i] = i;
    std::sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return probs[(size_t)a] > probs[(size_t)b]; });
    double entropy = 0.0;
    for (int i = 0; i < d.vocab_size; ++i)
      if (probs[(size_t)i] > 0.0f) entropy -= (double)probs[(size_t)i] * std::log((double)probs[(size_t)i]);
    std::ostringstream oss;
    oss << "[INFERENCE][INSPECT] Prompt=\"" << prompt << "\"\n";
    oss << "Argmax: id=" << order.front() << " token=\"" << tok.decode(order.front()) << "\"\n";
    oss << "Entropy: " << std::fixed << std::setprecision(6) << entropy << "\n";
    const size_t top = std::min<size_t>(5, order.size());
    oss << "Top-" << top << " next-token distribution:\n";
    for (size_t i = 0; i < top; ++i) {
      const int32_t id = order[i];
      oss << (i + 1) << ". id=" << id << " token=\"" << tok.decode(id) << "\" logit=" << std::fixed
          << std::setprecision(6) << logits[(size_t)id] << " prob=" << probs[(size_t)id] << "\n";
    }
    report("TOKEN_GEN", 0, 0.0f, oss.str());
  } else {
    api.destroy(s);
    throw std::runtime_error("unknown mode " + mode);
  }
  api.destroy(s);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  try {
    return run(argc, argv);
  } catch (const std::exception &e) {
    std::cerr << "litnice_b200_run: " << e.what() << "\n";
    return 1;
  }
}
