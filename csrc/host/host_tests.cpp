// Test program for the host runtime (csrc/host/*.hpp), meant to be built with the compiler's sanitizers:
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined -fno-sanitize-recover=undefined host_tests.cpp -pthread
//   g++ -std=c++17 -O1 -g -fsanitize=thread host_tests.cpp -pthread
// Usage: host_tests <scratch dir> [case ...]; without a case every one runs. Exit code 0 = all passed.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <functional>
#include <random>
#include <set>
#include <thread>

#include "paged_allocator.hpp"
#include "safetensors_map.hpp"
#include "signal_model.hpp"

using namespace cosmos::host;

#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) fail(__FILE__, ":", __LINE__, ": expectation failed: ", #cond); \
  } while (0)

template <typename F>
static bool throws_with(F&& f, const char* needle) {
  try {
    f();
  } catch (const std::runtime_error& e) {
    return std::string(e.what()).find(needle) != std::string::npos;
  }
  return false;
}

// ---------------------------------------------------------------- paged allocator
static void check_invariants(const PagedAllocator& a, const std::vector<int64_t>& live) {
  std::set<int32_t> seen;
  int64_t used = 0;
  for (int64_t s : live) {
    const auto* b = a.blocks(s);
    EXPECT(b != nullptr);
    EXPECT((int64_t)b->size() == (a.length(s) + a.block_size() - 1) / a.block_size());
    EXPECT((int64_t)b->size() <= a.max_blocks_per_seq());
    for (int32_t id : *b) {
      EXPECT(id >= 0 && id < a.num_blocks());
      EXPECT(seen.insert(id).second);  // no page belongs to two sequences
    }
    used += (int64_t)b->size();
  }
  EXPECT(used + a.num_free() == a.num_blocks());  // nothing leaks
}

static void test_allocator_random(const std::string&) {
  PagedAllocator a(97, 16, 12);
  std::mt19937 rng(7);
  std::vector<int64_t> live;
  int64_t next = 1;
  for (int it = 0; it < 20000; ++it) {
    const int op = (int)(rng() % 10);
    if (op < 2 || live.empty()) {  // new sequence with a prompt
      const int64_t tokens = 1 + (int64_t)(rng() % 150);
      const int64_t free_before = a.num_free();
      if (a.extend(next, tokens)) {
        live.push_back(next);
      } else {
        EXPECT(a.num_free() == free_before && a.blocks(next) == nullptr && a.length(next) == 0);  // failure changes nothing
      }
      ++next;
    } else if (op < 8) {  // decode: one more token
      const int64_t s = live[rng() % live.size()];
      const int64_t len = a.length(s), free_before = a.num_free();
      if (!a.extend(s, 1)) EXPECT(a.length(s) == len && a.num_free() == free_before);
    } else {  // retire
      const size_t i = rng() % live.size();
      a.release(live[i]);
      EXPECT(a.blocks(live[i]) == nullptr);
      live.erase(live.begin() + (long)i);
    }
    if (it % 97 == 0) check_invariants(a, live);
  }
  check_invariants(a, live);
  // table rows: -1 beyond the owned pages; unknown sequence gives an empty row
  std::vector<int64_t> q(live.begin(), live.begin() + (long)std::min<size_t>(live.size(), 5));
  q.push_back(-42);
  std::vector<int32_t> table(q.size() * 12, 7), lens(q.size(), 7);
  a.fill_tables(q.data(), (int64_t)q.size(), table.data(), lens.data());
  for (size_t i = 0; i < q.size(); ++i) {
    const auto* b = a.blocks(q[i]);
    const size_t nb = b ? b->size() : 0;
    EXPECT(lens[i] == (int32_t)a.length(q[i]));
    for (size_t j = 0; j < 12; ++j) EXPECT(table[i * 12 + j] == (j < nb ? (*b)[j] : -1));
  }
  for (int64_t s : live) a.release(s);
  EXPECT(a.num_free() == 97 && a.num_sequences() == 0);
  EXPECT(throws_with([] { PagedAllocator bad(0, 16, 4); }, "bad allocator sizes"));
}

// ---------------------------------------------------------------- safetensors mapping
static std::string write_file(const std::string& dir, const std::string& name, const std::string& header,
                              const std::string& data, int64_t claimed_header_len = -1) {
  const std::string path = dir + "/" + name;
  std::ofstream f(path, std::ios::binary);
  uint64_t n = claimed_header_len < 0 ? header.size() : (uint64_t)claimed_header_len;
  char len[8];
  for (int i = 0; i < 8; ++i) len[i] = (char)((n >> (8 * i)) & 0xff);
  f.write(len, 8);
  f.write(header.data(), (std::streamsize)header.size());
  f.write(data.data(), (std::streamsize)data.size());
  return path;
}

static void test_safetensors_valid_and_concurrent(const std::string& dir) {
  std::string data(4 * 6 + 2 * 4, '\0');
  for (int i = 0; i < 6; ++i) {
    float v = 0.5f * (float)i;
    std::memcpy(&data[4 * i], &v, 4);
  }
  for (int i = 0; i < 4; ++i) {
    uint16_t v = (uint16_t)(0x3f80 + i);
    std::memcpy(&data[24 + 2 * i], &v, 2);
  }
  const std::string header =
      "{\"__metadata__\":{\"format\":\"pt\",\"step\":\"12\",\"n\":3},"
      "\"a\":{\"dtype\":\"F32\",\"shape\":[2,3],\"data_offsets\":[0,24],\"extra\":{\"k\":[1,{\"z\":null}]}},"
      "\"b.w\":{\"dtype\":\"BF16\",\"shape\":[4],\"data_offsets\":[24,32]},"
      "\"empty\":{\"dtype\":\"I64\",\"shape\":[0,5],\"data_offsets\":[32,32]}}   ";
  const std::string path = write_file(dir, "ok.safetensors", header, data);
  SafetensorsMap m(path);
  EXPECT(m.keys().size() == 3 && m.keys()[0] == "a" && m.keys()[1] == "b.w");
  EXPECT(m.metadata().at("format") == "pt" && m.metadata().at("step") == "12" && m.metadata().count("n") == 0);
  EXPECT(m.find("a").numel == 6 && m.find("a").shape == (std::vector<int64_t>{2, 3}) && m.find("a").dtype == "F32");
  EXPECT(m.find("empty").numel == 0 && m.has("b.w") && !m.has("c"));
  float v4;
  std::memcpy(&v4, m.data("a", 4, 2), 4);
  EXPECT(v4 == 2.0f);
  EXPECT(throws_with([&] { m.data("a", 5, 2); }, "outside tensor 'a'"));
  EXPECT(throws_with([&] { m.data("a", -1, 1); }, "outside tensor"));
  EXPECT(throws_with([&] { m.find("nope"); }, "has no tensor 'nope'"));
  // The mapping is immutable: readers on several threads need no lock.
  std::vector<std::thread> ts;
  std::vector<double> sums(6, 0.0);
  for (int t = 0; t < 6; ++t)
    ts.emplace_back([&, t] {
      for (int rep = 0; rep < 200; ++rep) {
        double s = 0;
        for (int i = 0; i < 6; ++i) {
          float v;
          std::memcpy(&v, m.data("a", i, 1), 4);
          s += v;
        }
        sums[(size_t)t] = s;
      }
    });
  for (auto& t : ts) t.join();
  for (double s : sums) EXPECT(s == 7.5);
}

static void test_safetensors_rejects_bad_files(const std::string& dir) {
  const std::string d8(8, 'x');
  auto open = [&](const std::string& p) { SafetensorsMap m(p); };
  auto entry = [](const char* dtype, const char* shape, const char* offs) {
    return std::string("{\"t\":{\"dtype\":\"") + dtype + "\",\"shape\":" + shape + ",\"data_offsets\":" + offs + "}}";
  };
  EXPECT(throws_with([&] { open(dir + "/missing.safetensors"); }, "cannot open"));
  {
    std::ofstream f(dir + "/short.safetensors", std::ios::binary);
    f << "abc";
  }
  EXPECT(throws_with([&] { open(dir + "/short.safetensors"); }, "too short"));
  EXPECT(throws_with([&] { open(write_file(dir, "hdrlen.safetensors", "{}", "", 1 << 20)); }, "truncated or not a safetensors file"));
  EXPECT(throws_with([&] { open(write_file(dir, "trunc.safetensors", entry("F32", "[4]", "[0,16]"), d8)); }, "file truncated?"));
  EXPECT(throws_with([&] { open(write_file(dir, "span.safetensors", entry("F32", "[3]", "[0,8]"), d8)); }, "its shape and dtype need 12"));
  EXPECT(throws_with([&] { open(write_file(dir, "order.safetensors", entry("U8", "[0]", "[8,4]"), d8)); }, "offsets out of order"));
  EXPECT(throws_with([&] { open(write_file(dir, "dtype.safetensors", entry("F8_E4M3", "[8]", "[0,8]"), d8)); }, "unsupported dtype"));
  EXPECT(throws_with([&] { open(write_file(dir, "lacks.safetensors", "{\"t\":{\"dtype\":\"U8\",\"shape\":[8]}}", d8)); }, "lacks dtype"));
  EXPECT(throws_with([&] { open(write_file(dir, "ovf.safetensors", entry("F32", "[4611686018427387904,4]", "[0,8]"), d8)); }, "bad shape"));
  EXPECT(throws_with([&] { open(write_file(dir, "ovf2.safetensors", entry("U8", "[99999999999999999999]", "[0,8]"), d8)); }, "integer overflow"));
  EXPECT(throws_with([&] { open(write_file(dir, "dup.safetensors",
                                           "{\"t\":{\"dtype\":\"U8\",\"shape\":[8],\"data_offsets\":[0,8]},"
                                           "\"t\":{\"dtype\":\"U8\",\"shape\":[8],\"data_offsets\":[0,8]}}", d8)); }, "duplicate tensor"));
  EXPECT(throws_with([&] { open(write_file(dir, "json1.safetensors", "{\"t\":{\"dtype\":\"U8\",\"shape\":[8],\"data_offsets\":[0,8]}", d8)); }, "not valid JSON"));
  EXPECT(throws_with([&] { open(write_file(dir, "json2.safetensors", "{\"t\":{\"dtype\":\"U8", d8)); }, "not valid JSON"));
  EXPECT(throws_with([&] { open(write_file(dir, "json3.safetensors", "[1,2]", d8)); }, "not valid JSON"));
  std::string deep = "{\"t\":{\"dtype\":\"U8\",\"shape\":[8],\"data_offsets\":[0,8],\"x\":";
  for (int i = 0; i < 200; ++i) deep += "[";
  EXPECT(throws_with([&] { open(write_file(dir, "deep.safetensors", deep, d8)); }, "not valid JSON"));
  // random corruption of a valid header must end in an exception or a valid parse, never in a fault
  const std::string good = "{\"__metadata__\":{\"a\":\"b\"},\"t\":{\"dtype\":\"U8\",\"shape\":[2,4],\"data_offsets\":[0,8]}}";
  std::mt19937 rng(11);
  for (int it = 0; it < 400; ++it) {
    std::string h = good;
    const int edits = 1 + (int)(rng() % 3);
    for (int e = 0; e < edits; ++e) h[rng() % h.size()] = (char)(rng() % 256);
    if (rng() % 4 == 0) h.resize(rng() % h.size() + 1);
    try {
      SafetensorsMap m(write_file(dir, "fuzz.safetensors", h, d8));
      for (const auto& k : m.keys()) (void)m.data(k);
    } catch (const std::runtime_error&) {
    }
  }
}

// ---------------------------------------------------------------- signal-pad protocol
static void run_ranks(int world, const std::function<void(int)>& body) {
  std::vector<std::thread> ts;
  for (int r = 0; r < world; ++r) ts.emplace_back(body, r);
  for (auto& t : ts) t.join();
}

static void test_signal_allreduce_rounds(const std::string&) {
  const int world = 4, rounds = 300, slot = 3;
  const size_t n = 64;
  SignalWorld w(world, n);
  std::vector<int> bad(world, 0);
  run_ranks(world, [&](int r) {
    std::mt19937 rng((unsigned)r);
    std::vector<int64_t> out;
    for (int k = 1; k <= rounds; ++k) {
      if (rng() % 5 == 0) std::this_thread::yield();  // ranks drift apart
      for (size_t i = 0; i < n; ++i) w.inputs[(size_t)r][i] = (int64_t)k * 1000 + r * 10 + (int64_t)(i % 7);  // plain stores
      if (!allreduce_oneshot(w, r, slot, out, 1 << 26)) bad[(size_t)r]++;
      for (size_t i = 0; i < n; ++i) {
        const int64_t want = (int64_t)world * ((int64_t)k * 1000 + (int64_t)(i % 7)) + 10 * (world * (world - 1) / 2);
        if (out[i] != want) bad[(size_t)r]++;
      }
    }
  });
  for (int r = 0; r < world; ++r) {
    EXPECT(bad[(size_t)r] == 0);
    EXPECT(w.status[(size_t)r]->load() == kStatusOk);
    EXPECT(w.counters[(size_t)r][slot] == 2 * rounds);  // epoch counters stay in step with no argument changing
  }
}

static void test_signal_fast_rank_runs_one_barrier_ahead(const std::string&) {
  const int world = 3, slot = 0;
  SignalWorld w(world, 1);
  std::atomic<int> max_lead{0};
  std::vector<std::unique_ptr<std::atomic<int>>> at;
  for (int r = 0; r < world; ++r) at.emplace_back(new std::atomic<int>(0));
  run_ranks(world, [&](int r) {
    for (int e = 1; e <= 500; ++e) {
      at[(size_t)r]->store(e);
      const bool ok = barrier(w, r, slot, e, 1 << 26);
      if (!ok) std::abort();
      for (int p = 0; p < world; ++p) {
        const int seen = at[(size_t)p]->load();
        if (seen < e) std::abort();  // everybody reached epoch e before anyone left it
        int lead = seen - e, cur = max_lead.load();
        while (lead > cur && !max_lead.compare_exchange_weak(cur, lead)) {
        }
      }
    }
  });
  EXPECT(max_lead.load() <= 1);
}

static void test_signal_missing_peer_times_out(const std::string&) {
  const int world = 3;
  SignalWorld w(world, 1);
  std::vector<int> ok(world, 1);
  run_ranks(world, [&](int r) {
    if (r != 2) ok[(size_t)r] = barrier(w, r, 5, 1, 20000) ? 1 : 0;  // rank 2 never joins
  });
  for (int r = 0; r < 2; ++r) {
    EXPECT(ok[(size_t)r] == 0);  // the survivors give up instead of hanging
    EXPECT(w.status[(size_t)r]->load() == kStatusTimeoutPeer);
  }
  EXPECT(w.status[2]->load() == kStatusOk);
  // the status word keeps the first error
  EXPECT(!barrier(w, 0, 6, 1, 10, true));
  EXPECT(w.status[0]->load() == kStatusTimeoutPeer);
}

// Negative control, run only when named: without the trailing barrier a fast rank rewrites its input
// while a slow one still sums it. A thread sanitizer build must report this as a data race.
static void test_signal_without_trailing_barrier(const std::string&) {
  const int world = 2;
  SignalWorld w(world, 4096);
  run_ranks(world, [&](int r) {
    std::vector<int64_t> out;
    for (int k = 1; k <= 200; ++k) {
      for (auto& v : w.inputs[(size_t)r]) v = k;
      allreduce_oneshot(w, r, 1, out, 1 << 26, /*with_trailing_barrier=*/false);
    }
  });
}

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: %s <scratch dir> [case ...]\n", argv[0]);
    return 2;
  }
  const std::string dir = argv[1];
  const std::vector<std::pair<std::string, void (*)(const std::string&)>> cases = {
      {"allocator_random", test_allocator_random},
      {"safetensors_valid_and_concurrent", test_safetensors_valid_and_concurrent},
      {"safetensors_rejects_bad_files", test_safetensors_rejects_bad_files},
      {"signal_allreduce_rounds", test_signal_allreduce_rounds},
      {"signal_fast_rank_runs_one_barrier_ahead", test_signal_fast_rank_runs_one_barrier_ahead},
      {"signal_missing_peer_times_out", test_signal_missing_peer_times_out},
  };
  std::set<std::string> want(argv + 2, argv + argc);
  int failed = 0;
  if (want.count("signal_without_trailing_barrier")) {
    test_signal_without_trailing_barrier(dir);
    std::printf("DONE signal_without_trailing_barrier\n");
    want.erase("signal_without_trailing_barrier");
    if (want.empty()) return 0;
  }
  for (const auto& c : cases) {
    if (!want.empty() && !want.count(c.first)) continue;
    try {
      c.second(dir);
      std::printf("PASS %s\n", c.first.c_str());
    } catch (const std::exception& e) {
      std::printf("FAIL %s: %s\n", c.first.c_str(), e.what());
      ++failed;
    }
    std::fflush(stdout);
  }
  return failed ? 1 : 0;
}
