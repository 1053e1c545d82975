// Driver for the UNMODIFIED zscey/tiny-llm engine below its tokenizer: it does what the reference's
// Pipeline::apply does (tiny_llm/pipeline/pipeline.cpp:104-229) with token ids in place of text:
// llama_parser -> create_cuda_plan -> CudaRuntime, then set_prefill / bind_request_meta /
// cpu_tensor_copy_to_input / execute / output_copy_to_cpu_tensor and the reference's own ArgmaxProcessor
// on the host, in paged mode.  The tokenizer and the safetensors reader of the reference are Rust behind a
// C interface and cannot be built here, so weights come from a weight manager of this file (the
// reference's own tests do the same: tests/utils/weight_manager.hpp:8-63): either read from a
// model.safetensors in 32-bit, or drawn from a seed.  Everything that computes is the reference's code.
//
//   ref_driver bench  --config CONFIG.json --batch B --context C --steps K --warmup W [--repeats R] [--seed S]
//       B requests with prompts of C - (R*K + W) random tokens run as one prefill, then W + R*K decode steps;
//       prints one JSON line with the median time per step of the R timed runs of K steps.
//   ref_driver prefill --config CONFIG.json --tokens T [--repeats R]
//       one prompt of T tokens, R times; median time.
//   ref_driver logits --model DIR --tokens 1,2,3,... --decode N --out FILE
//       prompt whole, then N greedy tokens; writes the float32 logits of the prompt's last position and
//       of every decoded position ([1 + N, vocab]) and prints the chosen ids.
//   ref_driver graph --config CONFIG.json
//       prints the graph the reference's llama_parser builds (paged mode) as JSON: its nodes in order with
//       their kind and tensor names, and the tensors nothing produces (weights and inputs) with their shapes.
//       Needs no GPU.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <numeric>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "cuda_runtime.h"
#include "nlohmann/json.hpp"
#include "tiny_llm/device_managers/cuda/cuda_device_guard.hpp"
#include "tiny_llm/graph/graph.hpp"
#include "tiny_llm/logit_processors/argmax_processor.hpp"
#include "tiny_llm/parser/llama_parser.hpp"
#include "tiny_llm/runtime/cuda/cuda_runtime.hpp"
#include "tiny_llm/weight_managers/weight_managers.hpp"

namespace {
using tiny_llm::DataType;
using tiny_llm::Device;
using tiny_llm::DeviceType;
using tiny_llm::SliceView;
using tiny_llm::Tensor;

// Weights held on the host as float32, by checkpoint name.
class HostWeights {
public:
  HostWeights() = default;
  HostWeights(const HostWeights &) = delete;
  auto operator=(const HostWeights &) -> HostWeights & = delete;
  HostWeights(HostWeights &&) noexcept = default;
  auto operator=(HostWeights &&) noexcept -> HostWeights & = default;

  [[nodiscard]] auto get_tensor(const std::string &name) const -> SliceView {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) throw std::runtime_error("weight not found: " + name);
    return {DataType::kFloat32, it->second.first, it->second.second.data(), it->second.second.size() * sizeof(float)};
  }
  void set_tensor(std::string name, SliceView v) {
    std::vector<float> data(v.data_len / sizeof(float));
    std::memcpy(data.data(), v.data, v.data_len);
    tensors_[std::move(name)] = {v.shape, std::move(data)};
  }
  void put(std::string name, std::vector<int64_t> shape, std::vector<float> data) {
    tensors_[std::move(name)] = {std::move(shape), std::move(data)};
  }

private:
  std::unordered_map<std::string, std::pair<std::vector<int64_t>, std::vector<float>>> tensors_;
};

// xorshift64*: uniform in [-a, a] with standard deviation `std` (timing does not depend on the law)
struct Rng {
  uint64_t s;
  auto next() -> uint64_t {
    s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
    return s * 0x2545F4914F6CDD1DULL;
  }
  auto uniform(float a) -> float { return (static_cast<float>(next() >> 40) / 16777216.0F * 2.0F - 1.0F) * a; }
};

void fill_random(HostWeights &w, const std::string &name, std::vector<int64_t> shape, Rng &rng, float std_dev, bool ones = false) {
  size_t n = 1;
  for (auto d : shape) n *= static_cast<size_t>(d);
  std::vector<float> data(n);
  const float a = std_dev * 1.7320508F;
  for (auto &x : data) x = ones ? 1.0F : rng.uniform(a);
  w.put(name, std::move(shape), std::move(data));
}

auto random_weights(const nlohmann::json &c, uint64_t seed) -> HostWeights {
  HostWeights w;
  Rng rng{seed * 0x9E3779B97F4A7C15ULL + 1};
  const int64_t h = c["hidden_size"], inter = c["intermediate_size"], v = c["vocab_size"], layers = c["num_hidden_layers"];
  const int64_t nq = c["num_attention_heads"], nkv = c["num_key_value_heads"], hd = h / nq;
  const float s = 0.02F;
  fill_random(w, "model.embed_tokens.weight", {v, h}, rng, s);
  for (int64_t i = 0; i < layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    fill_random(w, p + "input_layernorm.weight", {h}, rng, s, true);
    fill_random(w, p + "self_attn.q_proj.weight", {nq * hd, h}, rng, s);
    fill_random(w, p + "self_attn.k_proj.weight", {nkv * hd, h}, rng, s);
    fill_random(w, p + "self_attn.v_proj.weight", {nkv * hd, h}, rng, s);
    fill_random(w, p + "self_attn.o_proj.weight", {h, nq * hd}, rng, s);
    fill_random(w, p + "post_attention_layernorm.weight", {h}, rng, s, true);
    fill_random(w, p + "mlp.gate_proj.weight", {inter, h}, rng, s);
    fill_random(w, p + "mlp.up_proj.weight", {inter, h}, rng, s);
    fill_random(w, p + "mlp.down_proj.weight", {h, inter}, rng, s);
  }
  fill_random(w, "model.norm.weight", {h}, rng, s, true);
  fill_random(w, "lm_head.weight", {v, h}, rng, s);
  return w;
}

// model.safetensors: 8 bytes little-endian header length, JSON header, data; 32-bit floats only (as the reference)
auto file_weights(const std::string &path) -> HostWeights {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  uint64_t n = 0;
  f.read(reinterpret_cast<char *>(&n), 8);
  std::string header(n, '\0');
  f.read(header.data(), static_cast<std::streamsize>(n));
  auto j = nlohmann::json::parse(header);
  HostWeights w;
  for (auto it = j.begin(); it != j.end(); ++it) {
    if (it.key() == "__metadata__") continue;
    if (it.value()["dtype"].get<std::string>() != "F32") throw std::runtime_error(it.key() + ": not F32");
    auto shape = it.value()["shape"].get<std::vector<int64_t>>();
    auto off = it.value()["data_offsets"].get<std::vector<uint64_t>>();
    std::vector<float> data((off[1] - off[0]) / 4);
    f.seekg(static_cast<std::streamoff>(8 + n + off[0]));
    f.read(reinterpret_cast<char *>(data.data()), static_cast<std::streamsize>(off[1] - off[0]));
    w.put(it.key(), std::move(shape), std::move(data));
  }
  return w;
}

struct Args {
  std::unordered_map<std::string, std::string> kv;
  auto get(const std::string &k, const std::string &d = "") const -> std::string {
    auto it = kv.find(k);
    return it == kv.end() ? d : it->second;
  }
  auto num(const std::string &k, long d) const -> long { return kv.count(k) ? std::stol(kv.at(k)) : d; }
};

// The engine below the tokenizer, as Pipeline's constructor sets it up (pipeline.cpp:45-97).
struct Engine {
  std::unique_ptr<tiny_llm::cuda::CudaRuntime> runtime;
  std::unique_ptr<Tensor> output;
  int64_t vocab{};
  uint32_t max_requests{};

  Engine(const nlohmann::json &config, HostWeights weights, uint32_t max_req) : max_requests(max_req) {
    const auto max_tokens = static_cast<uint32_t>(max_req * config["max_position_embeddings"].get<uint32_t>());
    auto plan = tiny_llm::cuda::create_cuda_plan(
        tiny_llm::llama_parser(config, true),
        {.named_shape_ranges = {{"token_ids", {.min_shape = {1, 1}, .max_shape = {1, max_tokens}}},
                                {"pos_ids", {.min_shape = {1, 1}, .max_shape = {1, max_tokens}}}}});
    tiny_llm::WeightManagerWrapper wm(std::move(weights));
    runtime = std::make_unique<tiny_llm::cuda::CudaRuntime>(std::move(plan), wm,
                                                            tiny_llm::cuda::RuntimeConfig{.max_request_num = max_req});
    vocab = config["vocab_size"].get<int64_t>();
    output = std::make_unique<Tensor>(Device{.type = DeviceType::kCudaHost, .id = 0}, DataType::kFloat32,
                                      std::vector<int64_t>{static_cast<int64_t>(max_req), 1, vocab});
  }

  // whole prompts in one step (pipeline.cpp:118-140)
  void prefill(const std::vector<std::vector<uint32_t>> &prompts, std::vector<tiny_llm::RequestMeta> &metas) {
    uint32_t total = 0;
    for (size_t i = 0; i < prompts.size(); ++i) {
      metas[i].seq_len = static_cast<uint32_t>(prompts[i].size());
      total += metas[i].seq_len;
    }
    Tensor token_ids({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {1, static_cast<int64_t>(total)});
    Tensor pos_ids({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {1, static_cast<int64_t>(total)});
    auto *t = token_ids.data<uint32_t>();
    auto *p = pos_ids.data<uint32_t>();
    for (const auto &r : prompts) {
      std::memcpy(t, r.data(), r.size() * sizeof(uint32_t));
      t += r.size();
      std::iota(p, p + r.size(), 0);
      p += r.size();
    }
    runtime->set_prefill(true);
    runtime->bind_request_meta(metas);
    runtime->cpu_tensor_copy_to_input("token_ids", token_ids);
    runtime->cpu_tensor_copy_to_input("pos_ids", pos_ids);
    runtime->execute();
    runtime->output_copy_to_cpu_tensor("lm_head.out", *output);
    for (auto &m : metas) m.seq_len = 1;
    runtime->set_prefill(false);
  }

  // one decode step (pipeline.cpp:183-191)
  void decode(std::vector<tiny_llm::RequestMeta> &metas, const Tensor &token_ids, const Tensor &pos_ids) {
    runtime->bind_request_meta(metas);
    runtime->cpu_tensor_copy_to_input("token_ids", token_ids);
    runtime->cpu_tensor_copy_to_input("pos_ids", pos_ids);
    runtime->execute();
    runtime->output_copy_to_cpu_tensor("lm_head.out", *output);
  }
};

// host sampling as the reference does it for do_sample = false (pipeline.cpp:193-226)
struct Greedy {
  Tensor indexes, valid, ids, pos;
  tiny_llm::ArgmaxProcessor argmax;
  int64_t batch, vocab;
  Greedy(int64_t b, int64_t v)
      : indexes({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {b, v}),
        valid({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {b}),
        ids({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {1, b}),
        pos({.type = DeviceType::kCpu, .id = 0}, DataType::kUint32, {1, b}), batch(b), vocab(v) {}
  void pick(Tensor &logits, const std::vector<uint32_t> &next_pos) {
    logits.reshape({batch, vocab});
    auto *ix = indexes.data<uint32_t>();
    auto *vs = valid.data<uint32_t>();
    for (int64_t i = 0; i < batch; ++i) {
      std::iota(ix + i * vocab, ix + (i + 1) * vocab, 0);
      vs[i] = static_cast<uint32_t>(vocab);
    }
    argmax.apply(logits, indexes, valid);
    for (int64_t i = 0; i < batch; ++i) {
      ids.data<uint32_t>()[i] = ix[i * vocab];
      pos.data<uint32_t>()[i] = next_pos[i];
    }
  }
};

auto median(std::vector<double> v) -> double {
  std::sort(v.begin(), v.end());
  return v[v.size() / 2];
}

auto run_bench(const Args &a) -> int {
  std::ifstream f(a.get("config"));
  auto config = nlohmann::json::parse(f);
  const auto batch = static_cast<int64_t>(a.num("batch", 8));
  const long context = a.num("context", 2048), steps = a.num("steps", 20), warmup = a.num("warmup", 3), repeats = a.num("repeats", 5);
  const long prompt_len = context - (repeats * steps + warmup);
  if (prompt_len < 1) throw std::runtime_error("steps do not fit the context");
  Engine eng(config, random_weights(config, static_cast<uint64_t>(a.num("seed", 2))), static_cast<uint32_t>(batch));
  Rng rng{12345};
  std::vector<std::vector<uint32_t>> prompts(batch, std::vector<uint32_t>(prompt_len));
  for (auto &p : prompts)
    for (auto &t : p) t = static_cast<uint32_t>(rng.next() % static_cast<uint64_t>(eng.vocab));
  std::vector<tiny_llm::RequestMeta> metas(batch);
  const auto p0 = std::chrono::steady_clock::now();
  eng.prefill(prompts, metas);
  const double prefill_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - p0).count();
  Greedy greedy(batch, eng.vocab);
  std::vector<uint32_t> next_pos(batch, static_cast<uint32_t>(prompt_len));
  auto step = [&] {
    greedy.pick(*eng.output, next_pos);
    eng.decode(metas, greedy.ids, greedy.pos);
    for (auto &p : next_pos) ++p;
  };
  for (long i = 0; i < warmup; ++i) step();
  std::vector<double> device_ms, wall_ms;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (long r = 0; r < repeats; ++r) {
    cudaDeviceSynchronize();
    const auto t0 = std::chrono::steady_clock::now();
    cudaEventRecord(e0, nullptr);
    for (long i = 0; i < steps; ++i) step();
    cudaEventRecord(e1, nullptr);
    cudaDeviceSynchronize();
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    device_ms.push_back(ms / static_cast<double>(steps));
    wall_ms.push_back(std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / static_cast<double>(steps));
  }
  eng.runtime->destroy_request_meta(metas);
  std::printf("{\"mode\": \"bench\", \"batch\": %ld, \"context\": %ld, \"steps\": %ld, \"warmup\": %ld, \"repeats\": %ld, "
              "\"ms_per_step_device\": %.4f, \"ms_per_step_wall\": %.4f, \"prefill_tokens\": %ld, \"prefill_ms_wall\": %.2f, "
              "\"h2d_bytes_per_step\": %ld, \"d2h_bytes_per_step\": %ld}\n",
              static_cast<long>(batch), context, steps, warmup, repeats, median(device_ms), median(wall_ms),
              static_cast<long>(batch) * prompt_len, prefill_ms, static_cast<long>(batch) * 8L, static_cast<long>(batch * eng.vocab * 4));
  return 0;
}

auto run_prefill(const Args &a) -> int {
  std::ifstream f(a.get("config"));
  auto config = nlohmann::json::parse(f);
  const long tokens = a.num("tokens", 2048), repeats = a.num("repeats", 3);
  Engine eng(config, random_weights(config, static_cast<uint64_t>(a.num("seed", 2))), 1);
  Rng rng{777};
  std::vector<std::vector<uint32_t>> prompts(1, std::vector<uint32_t>(tokens));
  for (auto &t : prompts[0]) t = static_cast<uint32_t>(rng.next() % static_cast<uint64_t>(eng.vocab));
  std::vector<double> ms;
  for (long r = 0; r < repeats + 1; ++r) {
    std::vector<tiny_llm::RequestMeta> metas(1);
    cudaDeviceSynchronize();
    const auto t0 = std::chrono::steady_clock::now();
    eng.prefill(prompts, metas);
    cudaDeviceSynchronize();
    if (r > 0) ms.push_back(std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
    eng.runtime->destroy_request_meta(metas);
  }
  std::printf("{\"mode\": \"prefill\", \"tokens\": %ld, \"ms\": %.3f}\n", tokens, median(ms));
  return 0;
}

auto run_graph(const Args &a) -> int {
  std::ifstream f(a.get("config"));
  auto config = nlohmann::json::parse(f);
  const tiny_llm::Graph g = tiny_llm::llama_parser(config, true);
  static const char *kinds[] = {"silu", "embedding", "rope", "rms_norm", "add", "mul", "linear", "causal_attention", "slice_linear"};
  nlohmann::json out;
  out["valid"] = tiny_llm::is_valid(g);
  auto names = [&g](const std::vector<uint32_t> &ids) {
    std::vector<std::string> r;
    for (auto id : ids) r.push_back(g.tensor_infos.at(id)->first);
    return r;
  };
  out["nodes"] = nlohmann::json::array();
  for (const auto &n : g.nodes) {
    if (!n) continue;
    out["nodes"].push_back({{"name", n->first}, {"kind", kinds[n->second.param.index()]},
                            {"inputs", names(n->second.input_tensors)}, {"outputs", names(n->second.output_tensors)}});
  }
  out["sources"] = nlohmann::json::object();
  for (const auto &t : g.tensor_infos)
    if (t && !t->second.producer_node) out["sources"][t->first] = t->second.shape;
  out["inputs"] = std::vector<std::string>(g.input_names.begin(), g.input_names.end());
  out["outputs"] = std::vector<std::string>(g.output_names.begin(), g.output_names.end());
  std::cout << out.dump() << "\n";
  return 0;
}

auto run_logits(const Args &a) -> int {
  const std::string dir = a.get("model");
  std::ifstream f(dir + "/config.json");
  auto config = nlohmann::json::parse(f);
  std::vector<uint32_t> prompt;
  std::stringstream ss(a.get("tokens"));
  for (std::string tok; std::getline(ss, tok, ',');) prompt.push_back(static_cast<uint32_t>(std::stoul(tok)));
  const long n_decode = a.num("decode", 4);
  Engine eng(config, file_weights(dir + "/model.safetensors"), 1);
  std::vector<tiny_llm::RequestMeta> metas(1);
  eng.prefill({prompt}, metas);
  Greedy greedy(1, eng.vocab);
  std::ofstream out(a.get("out"), std::ios::binary);
  std::vector<uint32_t> next_pos(1, static_cast<uint32_t>(prompt.size()));
  std::printf("{\"mode\": \"logits\", \"ids\": [");
  for (long i = 0; i <= n_decode; ++i) {
    out.write(reinterpret_cast<const char *>(eng.output->data<float>()), static_cast<std::streamsize>(eng.vocab * 4));
    if (i == n_decode) break;
    greedy.pick(*eng.output, next_pos);     // (moves the chosen id to the front of the index row; the logits were written before)
    std::printf("%s%u", i ? ", " : "", greedy.ids.data<uint32_t>()[0]);
    eng.decode(metas, greedy.ids, greedy.pos);
    ++next_pos[0];
  }
  std::printf("]}\n");
  eng.runtime->destroy_request_meta(metas);
  return 0;
}
}  // namespace

auto main(int argc, char **argv) -> int {
  if (argc < 2) {
    std::cerr << "usage: ref_driver bench|prefill|logits --key value ...\n";
    return 2;
  }
  Args a;
  for (int i = 2; i + 1 < argc; i += 2) a.kv[std::string(argv[i]).substr(2)] = argv[i + 1];
  try {
    const std::string mode = argv[1];
    if (mode == "graph") return run_graph(a);
    tiny_llm::CudaDeviceSwitchGuard guard(static_cast<tiny_llm::DeviceId>(a.num("device", 0)));
    if (mode == "bench") return run_bench(a);
    if (mode == "prefill") return run_prefill(a);
    if (mode == "logits") return run_logits(a);
    std::cerr << "unknown mode " << mode << "\n";
    return 2;
  } catch (const std::exception &e) {
    std::cerr << "[ref_driver] " << e.what() << "\n";
    return 1;
  }
}
