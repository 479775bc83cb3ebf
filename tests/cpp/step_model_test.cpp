// The reference's UNMODIFIED engine (src/engine/engine.cpp + sampler.cpp, compiled where they lie) driving the GPU
// path through the reference's own scheduler <-> model interface: PkvStepModel (unholy_b200/csrc/host/step_model.hpp)
// implements StepModel (src/engine/step.hpp:76-106) on libunholy_pkv.so. The method is the reference's scheduler test
// (tools/sched_test/main.cpp): the model keeps a paged token store addressed only through the engine's block tables
// and answers with one-hot logits of a hash of the whole sequence read back through the table — here the store is a
// row pool in HBM written by pkv_step_run and read back by its gather. Greedy outputs of every request must equal a
// standalone simulation of the same hash chain, through prefix hits (shared pages + restored slot state), recompute
// preemption (a pool too small for the running set), aborts and two steps in flight; no page may leak. Prints and
// returns non-zero on failure. Built by oracle/build_oracle.py into oracle/_ref/ (it contains the reference's engine);
// run by tests/test_gpu_step_model.py.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <random>
#include <vector>

#include "engine/engine.hpp"
#include "../../unholy_b200/csrc/host/step_model.hpp"

using namespace unholy::engine;

namespace {
constexpr int kVocab = 512, kEos = 1;

uint64_t chain(const std::vector<int32_t>& seq) {
  uint64_t h = 1469598103934665603ull;
  for (const int32_t t : seq) h = (h ^ uint64_t(uint32_t(t))) * 1099511628211ull;
  return h;
}
int32_t next_token(const std::vector<int32_t>& seq) {
  const uint64_t h = chain(seq);
  if (h % 61 == 0) return kEos;
  return int32_t(2 + (h >> 9) % (kVocab - 2));
}
// What a correct model + engine must produce for a prompt: the hash chain followed until EOS or a length limit.
std::vector<int32_t> simulate(std::vector<int32_t> seq, int max_tokens, int max_context, FinishReason& why) {
  std::vector<int32_t> out;
  for (;;) {
    const int32_t t = next_token(seq);
    if (t == kEos) {
      why = FinishReason::Stop;
      return out;
    }
    seq.push_back(t);
    out.push_back(t);
    if ((max_tokens > 0 && int(out.size()) >= max_tokens) || int(seq.size()) >= max_context) {
      why = FinishReason::Length;
      return out;
    }
  }
}

struct Got {
  std::vector<int32_t> tokens;
  bool finished = false;
  FinishReason why = FinishReason::None;
  int cached = 0;
  std::string error;
};

struct Scenario {
  const char* name;
  int slots, pages_per_seq, pages, page_tokens, budget, inflight, snapshots, requests;
  bool bulk, aborts;
  int decode_pages;  // longest completion, in pages
  bool want_preemptions;
};

int run(const Scenario& sc) {
  unholy::kernels::PkvStepModel model(kVocab, sc.slots, sc.pages_per_seq, sc.pages, sc.page_tokens, sc.budget, 64, sc.inflight,
                                      sc.snapshots, next_token);
  model.use_bulk_pipeline(sc.bulk);
  EngineConfig cfg;
  cfg.max_batch_tokens = sc.budget;
  cfg.eos_id = kEos;
  Engine eng(model, cfg, false);
  std::mt19937_64 rng(std::hash<std::string>{}(sc.name));
  const auto rnd = [&](int lo, int hi) { return lo + int(rng() % uint64_t(hi - lo + 1)); };
  // a few shared prefixes (several pages long) so that later requests hit the prefix cache
  std::vector<std::vector<int32_t>> prefixes(4);
  for (auto& p : prefixes) {
    p.resize(size_t(rnd(3, 9) * sc.page_tokens + rnd(0, sc.page_tokens - 1)));
    for (auto& t : p) t = rnd(2, kVocab - 1);
  }
  std::map<uint64_t, Got> got;
  std::map<uint64_t, std::pair<std::vector<int32_t>, int>> asked;  // id -> (prompt, max_tokens)
  std::vector<uint64_t> aborted;
  int submitted = 0, fails = 0;
  // Requests arrive over time; the sink records what each one produced.
  const auto submit_request = [&]() {
    GenRequest r;
    if (rnd(0, 2) != 0) r.prompt = prefixes[size_t(rnd(0, 3))];
    const int extra = rnd(1, 3 * sc.page_tokens);
    for (int i = 0; i < extra; ++i) r.prompt.push_back(rnd(2, kVocab - 1));
    r.max_tokens = rnd(1, sc.decode_pages * sc.page_tokens);
    r.sampling.temperature = 0.0f;
    auto prompt = r.prompt;
    const int mt = r.max_tokens;
    auto key = std::make_shared<uint64_t>(0);
    const uint64_t id = eng.submit(std::move(r), [&got, key](GenOutput&& o) {
      Got& g = got[*key];
      g.tokens.insert(g.tokens.end(), o.tokens.begin(), o.tokens.end());
      g.cached = o.cached_tokens;
      if (o.finished) g.finished = true, g.why = o.reason, g.error = o.error;
    });
    *key = id;
    asked[id] = {std::move(prompt), mt};
    ++submitted;
  };
  int iterations = 0;
  while (submitted < sc.requests || eng.stats().running + eng.stats().waiting > 0) {
    if (submitted < sc.requests && rnd(0, 3) == 0) submit_request();
    if (sc.aborts && !asked.empty() && rnd(0, 40) == 0) {  // a client goes away
      auto it = asked.begin();
      std::advance(it, rnd(0, int(asked.size()) - 1));
      if (!got[it->first].finished) {
        eng.abort(it->first);
        aborted.push_back(it->first);
      }
    }
    eng.iterate();
    if (++iterations > 2000000) {
      std::printf("%s: the engine did not drain\n", sc.name);
      return 1;
    }
  }
  for (int i = 0; i < 4; ++i) eng.iterate();
  const EngineStats st = eng.stats();
  long cached_total = 0;
  int checked = 0;
  for (const auto& kv : asked) {
    const Got& g = got[kv.first];
    const bool was_aborted = std::find(aborted.begin(), aborted.end(), kv.first) != aborted.end();
    if (!g.finished) {
      std::printf("%s: request %llu never finished\n", sc.name, (unsigned long long)kv.first);
      ++fails;
      continue;
    }
    FinishReason why = FinishReason::None;
    const std::vector<int32_t> want = simulate(kv.second.first, kv.second.second, eng.max_context(), why);
    if (was_aborted && g.why == FinishReason::Abort) {  // what it produced before the abort must be a prefix of the truth
      if (g.tokens.size() > want.size() || !std::equal(g.tokens.begin(), g.tokens.end(), want.begin())) {
        std::printf("%s: aborted request %llu produced tokens off the chain\n", sc.name, (unsigned long long)kv.first);
        ++fails;
      }
      continue;
    }
    if (!g.error.empty() || g.tokens != want || g.why != why) {
      std::printf("%s: request %llu differs from the simulation (%zu vs %zu tokens, error '%s')\n", sc.name,
                  (unsigned long long)kv.first, g.tokens.size(), want.size(), g.error.c_str());
      ++fails;
    }
    cached_total += g.cached;
    ++checked;
  }
  if (st.free_pages != st.total_pages) {  // tools/sched_test/main.cpp:1113-1116
    std::printf("%s: %d of %d pages are still held after every request finished\n", sc.name, st.total_pages - st.free_pages, st.total_pages);
    ++fails;
  }
  std::printf("%s: %d requests checked (%zu aborted), %llu steps, %llu preemptions, %ld prompt tokens served from shared pages, %d failures\n",
              sc.name, checked, aborted.size(), (unsigned long long)st.steps, (unsigned long long)st.preemptions, cached_total, fails);
  if (sc.snapshots > 0 && cached_total == 0) {
    std::printf("%s: expected prefix hits\n", sc.name);
    ++fails;
  }
  if (sc.want_preemptions && st.preemptions == 0) {
    std::printf("%s: expected recompute preemptions\n", sc.name);
    ++fails;
  }
  return fails;
}
}  // namespace

int main() {
  int fails = 0;
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) {
    std::printf("no CUDA device\n");
    return 2;
  }
  const Scenario scenarios[] = {
      //  name                     slots pps pages page budget inflight snaps requests bulk  aborts
      {"roomy pool, prefix cache", 8, 64, 512, 16, 256, 1, 32, 60, false, false, 4, false},
      {"tight pool (preemption)", 6, 48, 44, 16, 128, 1, 0, 50, false, false, 14, true},
      {"tight pool, prefix cache, two in flight", 6, 48, 52, 16, 128, 2, 16, 60, false, true, 12, true},
      {"two in flight + aborts", 8, 64, 192, 16, 192, 2, 24, 70, false, true, 4, false},
      {"bulk pipeline", 8, 64, 256, 16, 256, 2, 16, 40, true, true, 4, false},
      {"small pages", 4, 128, 160, 8, 96, 1, 64, 50, false, false, 6, false},
  };
  for (const Scenario& sc : scenarios) {
    try {
      fails += run(sc);
    } catch (const std::exception& e) {
      std::printf("%s: exception: %s\n", sc.name, e.what());
      ++fails;
    }
  }
  std::printf(fails ? "FAILED\n" : "all ok\n");
  return fails ? 1 : 0;
}
