// Self-test of the host I/O runtime core (io_core.h) as a plain program, meant to be built with
// -fsanitize=address,undefined and with -fsanitize=thread:
//     g++ -std=c++17 -O1 -g -pthread -fsanitize=address,undefined -fno-sanitize-recover=all io_selftest.cpp -o t && ./t DIR
// Exercises: many concurrent writer jobs from two submitting threads (+ error reporting for an unwritable path),
// the mmap gatherer over several part files of every token width against a flat copy, the sample index against a
// brute-force walk, and the blend index against its defining property.  Exit code 0 = every check passed.
#include "io_core.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <fstream>
#include <random>

namespace {

int g_failures = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) {                                                           \
      std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond); \
      ++g_failures;                                                          \
    }                                                                        \
  } while (0)

std::vector<char> read_file(const std::string& p) {
  std::ifstream f(p, std::ios::binary);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

void test_writer(const std::string& dir) {
  constexpr int kJobs = 64;
  std::vector<std::shared_ptr<std::vector<char>>> bufs;
  std::mt19937 rng(1);
  for (int i = 0; i < kJobs; ++i) {
    auto b = std::make_shared<std::vector<char>>(static_cast<size_t>(1000 + 37 * i));
    for (auto& c : *b) c = static_cast<char>(rng());
    bufs.push_back(b);
  }
  {
    mtio::AsyncFileWriter w(4);
    auto submit_range = [&](int lo, int hi) {
      for (int i = lo; i < hi; ++i)
        w.submit(dir + "/f" + std::to_string(i) + ".bin", bufs[i]->data(), bufs[i]->size(), bufs[i]);
    };
    std::thread other(submit_range, kJobs / 2, kJobs);  // two submitters race on the queue
    submit_range(0, kJobs / 2);
    other.join();
    w.wait();
    CHECK(w.pending() == 0);
    for (int i = 0; i < kJobs; ++i) CHECK(read_file(dir + "/f" + std::to_string(i) + ".bin") == *bufs[i]);
    // an unwritable path is reported by wait(), once
    w.submit(dir + "/no_such_dir/x.bin", bufs[0]->data(), bufs[0]->size(), bufs[0]);
    bool threw = false;
    try {
      w.wait();
    } catch (const std::runtime_error&) {
      threw = true;
    }
    CHECK(threw);
    w.wait();  // the error was consumed
    // jobs still queued when the writer is destroyed are written before the workers exit
    for (int i = 0; i < 8; ++i) w.submit(dir + "/late" + std::to_string(i) + ".bin", bufs[i]->data(), bufs[i]->size(), bufs[i]);
  }
  for (int i = 0; i < 8; ++i) CHECK(read_file(dir + "/late" + std::to_string(i) + ".bin") == *bufs[i]);
}

template <typename T>
void test_mmap_width(const std::string& dir) {
  std::mt19937 rng(static_cast<unsigned>(sizeof(T)));
  std::vector<T> all;
  std::vector<std::string> paths;
  const int part_tokens[4] = {100, 1, 0, 257};  // one empty part
  for (int p = 0; p < 4; ++p) {
    std::vector<T> part(static_cast<size_t>(part_tokens[p]));
    for (auto& t : part) t = static_cast<T>(rng() % 30000);
    const std::string path = dir + "/tok" + std::to_string(sizeof(T)) + "_" + std::to_string(p) + ".bin";
    std::ofstream(path, std::ios::binary).write(reinterpret_cast<const char*>(part.data()), part.size() * sizeof(T));
    paths.push_back(path);
    all.insert(all.end(), part.begin(), part.end());
  }
  mtio::MMapTokens m(paths, static_cast<int64_t>(sizeof(T)));
  CHECK(m.total_bytes() == static_cast<int64_t>(all.size() * sizeof(T)));
  const int64_t offs[3] = {95 * static_cast<int64_t>(sizeof(T)), 0, 300 * static_cast<int64_t>(sizeof(T))};
  const int64_t cnts[3] = {20, 5, 58};  // the first span crosses three parts, the last ends at the last token
  std::vector<int32_t> out(90, -1);
  m.gather(offs, cnts, 3, out.data(), static_cast<int64_t>(out.size()));
  int64_t pos = 0;
  for (int s = 0; s < 3; ++s)
    for (int64_t t = 0; t < cnts[s]; ++t, ++pos)
      CHECK(out[static_cast<size_t>(pos)] == static_cast<int32_t>(all[static_cast<size_t>(offs[s] / sizeof(T) + t)]));
  for (; pos < 90; ++pos) CHECK(out[static_cast<size_t>(pos)] == 0);
  bool threw = false;
  const int64_t bad_off[1] = {static_cast<int64_t>(all.size() * sizeof(T))}, one[1] = {1};
  try {
    m.gather(bad_off, one, 1, out.data(), 4);
  } catch (const std::out_of_range&) {
    threw = true;
  }
  CHECK(threw);
}

void test_sample_index() {
  std::mt19937 rng(3);
  for (int trial = 0; trial < 50; ++trial) {
    const int n = 1 + static_cast<int>(rng() % 40);
    std::vector<int64_t> lens(static_cast<size_t>(n)), order(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) {
      lens[i] = static_cast<int64_t>(rng() % 25);  // zero-length documents included
      order[i] = i;
    }
    std::shuffle(order.begin(), order.end(), rng);
    const int64_t target = 1 + static_cast<int64_t>(rng() % 17);
    const auto rows = mtio::build_sample_index(lens.data(), order.data(), n, target);
    int64_t total = 0;
    for (int i = 0; i < n; ++i) total += lens[i];
    CHECK(static_cast<int64_t>(rows.size() / 2) == total / target + 1);
    // every boundary, translated to a position in the concatenated stream, is a multiple of the sample length
    std::vector<int64_t> start(static_cast<size_t>(n) + 1, 0);
    for (int i = 0; i < n; ++i) start[i + 1] = start[i] + lens[order[i]];
    for (size_t r = 0; r < rows.size() / 2; ++r) {
      CHECK(rows[2 * r] >= 0 && rows[2 * r] < n);
      CHECK(rows[2 * r + 1] >= 0 && rows[2 * r + 1] <= lens[order[rows[2 * r]]]);
      CHECK(start[rows[2 * r]] + rows[2 * r + 1] == static_cast<int64_t>(r) * target);
    }
  }
}

void test_blend_index() {
  const double w[3] = {0.5, 0.3, 0.2};
  const int64_t len[3] = {7, 1000, 3};
  constexpr int64_t size = 1000;
  std::vector<int32_t> ds(size);
  std::vector<int64_t> si(size);
  mtio::build_blend_index(w, len, 3, size, ds.data(), si.data());
  int64_t counts[3] = {0, 0, 0};
  for (int64_t i = 0; i < size; ++i) {
    CHECK(ds[i] >= 0 && ds[i] < 3);
    CHECK(si[i] == counts[ds[i]] % len[ds[i]]);
    ++counts[ds[i]];
    for (int k = 0; k < 3; ++k) CHECK(std::abs(static_cast<double>(counts[k]) - w[k] * (i + 1)) <= 1.0 + 1e-9);
  }
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: %s <scratch directory>\n", argv[0]);
    return 2;
  }
  const std::string dir = argv[1];
  test_writer(dir);
  test_mmap_width<uint8_t>(dir);
  test_mmap_width<uint16_t>(dir);
  test_mmap_width<int32_t>(dir);
  test_mmap_width<int64_t>(dir);
  test_sample_index();
  test_blend_index();
  if (g_failures == 0) std::printf("io_selftest: all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
