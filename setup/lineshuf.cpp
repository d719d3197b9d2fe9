// lineshuf: shuffle the lines of a text stream that may be larger than memory.
//
//   MEMORY=4 SEED=42 TMPDIR=/scratch ./lineshuf < in.jsonl > out.jsonl
//
// The role terashuf plays in the reference's data preparation (setup/download_prepare_hf_data.py:65-76,
// 128-133), as a small in-tree tool. Pass 1 reads as many lines as fit in MEMORY gigabytes, shuffles them and
// writes them to a temporary file; repeat until the input ends. Pass 2 draws the next output line from
// temporary file i with probability (lines left in i) / (lines left in total) and streams it out, which makes
// every permutation of the input equally likely. With a single chunk nothing touches the disk.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>
#include <unistd.h>

struct Chunk {
  std::string path;
  FILE* f = nullptr;
  uint64_t left = 0;
};

static bool read_line(FILE* f, std::string& out) {
  out.clear();
  char buf[1 << 16];
  while (fgets(buf, sizeof buf, f)) {
    out += buf;
    if (!out.empty() && out.back() == '\n') return true;
  }
  if (out.empty()) return false;
  out += '\n';  // last line without a terminator
  return true;
}

int main() {
  const char* mem_env = getenv("MEMORY");
  const char* seed_env = getenv("SEED");
  const char* tmp_env = getenv("TMPDIR");
  const double mem_gb = mem_env ? atof(mem_env) : 4.0;
  const uint64_t budget = static_cast<uint64_t>(mem_gb * (1ull << 30));
  std::mt19937_64 rng(seed_env ? strtoull(seed_env, nullptr, 10) : 42ull);
  const std::string tmpdir = tmp_env ? tmp_env : "/tmp";

  std::vector<Chunk> chunks;
  std::string data;                // lines of the current chunk, back to back
  std::vector<uint64_t> starts;    // offset of every line in `data`
  std::string line;
  bool more = true;
  auto flush_chunk = [&](bool to_stdout) {
    std::vector<uint32_t> order(starts.size());
    for (uint32_t i = 0; i < order.size(); ++i) order[i] = i;
    std::shuffle(order.begin(), order.end(), rng);
    FILE* out = stdout;
    Chunk c;
    if (!to_stdout) {
      c.path = tmpdir + "/lineshuf." + std::to_string(getpid()) + "." + std::to_string(chunks.size());
      out = fopen(c.path.c_str(), "wb");
      if (!out) { perror("lineshuf: cannot create temporary file"); exit(1); }
    }
    for (uint32_t i : order) {
      const uint64_t b = starts[i], e = (i + 1 < starts.size()) ? starts[i + 1] : data.size();
      fwrite(data.data() + b, 1, e - b, out);
    }
    if (!to_stdout) {
      fclose(out);
      c.left = starts.size();
      chunks.push_back(c);
    }
    data.clear();
    starts.clear();
  };
  while (more) {
    more = read_line(stdin, line);
    if (more) {
      starts.push_back(data.size());
      data += line;
    }
    if (!more || data.size() + starts.size() * 12 >= budget) {
      if (!more && chunks.empty()) {  // everything fitted: no temporary files at all
        flush_chunk(true);
        return 0;
      }
      if (!starts.empty()) flush_chunk(false);
    }
  }
  uint64_t total = 0;
  for (auto& c : chunks) {
    c.f = fopen(c.path.c_str(), "rb");
    if (!c.f) { perror("lineshuf: cannot reopen temporary file"); return 1; }
    total += c.left;
  }
  while (total > 0) {
    uint64_t pick = std::uniform_int_distribution<uint64_t>(0, total - 1)(rng);
    size_t i = 0;
    while (pick >= chunks[i].left) pick -= chunks[i++].left;
    if (!read_line(chunks[i].f, line)) { fprintf(stderr, "lineshuf: temporary file ended early\n"); return 1; }
    fwrite(line.data(), 1, line.size(), stdout);
    --chunks[i].left;
    --total;
  }
  for (auto& c : chunks) {
    fclose(c.f);
    remove(c.path.c_str());
  }
  return 0;
}
