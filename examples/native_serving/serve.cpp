// Stand-alone serving program without Python (the role of examples/online_serving/main.cc in the reference, which
// links an AOT-compiled dense graph and fakes the sparse lookup).  This one looks the ids up for real:
//
//   dictionary : text file `sign \t w0 \t w1 ...` (optionally with [ ] around the weights, optionally gzip), as written
//                by `python -m tensornet_b200.tools merge-sparse` / `tn.serving.export_sparse_dictionary`
//   tower      : binary file written by `tn.serving.export_tower(mlp, head, path)`:
//                "TNTW0001" | u32 layers | per layer: u32 out, u32 in, u32 relu, float32 W[out][in], float32 b[out]
//   request    : ids [slots][batch]; every slot's vector is looked up (zeros when unknown), the slots are
//                concatenated per example, the tower runs in fp32 and a sigmoid gives the click probability.
//
//   g++ -O3 -std=c++17 -pthread examples/native_serving/serve.cpp -lz -o /tmp/tn_serve
//   /tmp/tn_serve --dict deep_input.dict.txt --tower tower.bin --slots 4 --dim 8 --batch 32 --requests 1000
//   /tmp/tn_serve --dict ... --tower ... --slots 4 --dim 8 --ids request.txt --dump       # S lines of B ids -> probabilities
//
// It is the CPU counterpart of `tn.serving.InferenceEngine`; on a GPU the same files are served by that class
// (hash table probed by a kernel, towers on the tensor cores, one CUDA graph per batch shape).
#include <zlib.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

struct Dictionary {
  int dim = 0;
  std::vector<uint64_t> keys;      // open addressing, 0 = empty (sign 0 is kept aside)
  std::vector<int32_t> slot;
  std::vector<float> rows;
  std::vector<uint64_t> all_signs;
  int64_t zero_row = -1;
  uint64_t mask = 0;

  static uint64_t mix(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
    return x;
  }

  void load(const std::string& path, int want_dim) {
    gzFile f = gzopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    gzbuffer(f, 1 << 20);
    dim = want_dim;
    std::vector<char> line(1 << 16);
    std::vector<std::pair<uint64_t, int64_t>> entries;
    while (gzgets(f, line.data(), (int)line.size())) {
      char* p = line.data();
      char* end = nullptr;
      const uint64_t sign = std::strtoull(p, &end, 10);
      if (end == p) continue;
      const int64_t row = (int64_t)(rows.size() / dim);
      rows.resize(rows.size() + dim, 0.f);
      p = end;
      for (int k = 0; k < dim; ++k) {
        while (*p == '\t' || *p == ' ' || *p == '[' || *p == ',') ++p;
        if (*p == '\0' || *p == '\n' || *p == ']') break;
        rows[(size_t)row * dim + k] = std::strtof(p, &end);
        if (end == p) break;
        p = end;
      }
      entries.emplace_back(sign, row);
      all_signs.push_back(sign);
    }
    gzclose(f);
    size_t cap = 16;
    while (cap < entries.size() * 2 + 1) cap <<= 1;
    mask = cap - 1;
    keys.assign(cap, 0);
    slot.assign(cap, -1);
    for (auto& e : entries) {
      if (e.first == 0) { zero_row = e.second; continue; }
      uint64_t h = mix(e.first) & mask;
      while (keys[h] != 0 && keys[h] != e.first) h = (h + 1) & mask;
      keys[h] = e.first;
      slot[h] = (int32_t)e.second;            // a sign listed twice: the later line wins
    }
  }

  const float* find(uint64_t sign) const {
    if (sign == 0) return zero_row < 0 ? nullptr : rows.data() + (size_t)zero_row * dim;
    uint64_t h = mix(sign) & mask;
    while (keys[h] != 0) {
      if (keys[h] == sign) return rows.data() + (size_t)slot[h] * dim;
      h = (h + 1) & mask;
    }
    return nullptr;
  }
};

struct Layer {
  uint32_t out = 0, in = 0, relu = 0;
  std::vector<float> w, b;
};

static std::vector<Layer> load_tower(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  char magic[8];
  uint32_t n = 0;
  f.read(magic, 8);
  f.read(reinterpret_cast<char*>(&n), 4);
  if (!f || std::memcmp(magic, "TNTW0001", 8) != 0 || n == 0 || n > 64) throw std::runtime_error(path + " is not a tower file");
  std::vector<Layer> layers(n);
  for (auto& l : layers) {
    f.read(reinterpret_cast<char*>(&l.out), 4);
    f.read(reinterpret_cast<char*>(&l.in), 4);
    f.read(reinterpret_cast<char*>(&l.relu), 4);
    if (!f || l.out == 0 || l.in == 0 || (uint64_t)l.out * l.in > (1ull << 30)) throw std::runtime_error(path + " is damaged");
    l.w.resize((size_t)l.out * l.in);
    l.b.resize(l.out);
    f.read(reinterpret_cast<char*>(l.w.data()), (std::streamsize)(l.w.size() * 4));
    f.read(reinterpret_cast<char*>(l.b.data()), (std::streamsize)(l.b.size() * 4));
    if (!f) throw std::runtime_error(path + " ends early");
  }
  for (size_t i = 1; i < layers.size(); ++i)
    if (layers[i].in != layers[i - 1].out) throw std::runtime_error("layer widths of " + path + " do not chain");
  return layers;
}

// ids [S][B] -> probabilities [B]
static void infer(const Dictionary& d, const std::vector<Layer>& tower, const uint64_t* ids, int S, int B, std::vector<float>& x,
                  std::vector<float>& y, float* prob) {
  const int dim = d.dim, width = S * dim;
  x.assign((size_t)B * width, 0.f);
  for (int s = 0; s < S; ++s)
    for (int b = 0; b < B; ++b)
      if (const float* row = d.find(ids[(size_t)s * B + b])) std::memcpy(&x[(size_t)b * width + (size_t)s * dim], row, (size_t)dim * 4);
  int in = width;
  for (const Layer& l : tower) {
    y.assign((size_t)B * l.out, 0.f);
    for (int b = 0; b < B; ++b) {
      const float* xb = &x[(size_t)b * in];
      float* yb = &y[(size_t)b * l.out];
      for (uint32_t o = 0; o < l.out; ++o) {
        const float* w = &l.w[(size_t)o * l.in];
        float acc = l.b[o];
        for (uint32_t k = 0; k < l.in; ++k) acc += w[k] * xb[k];
        yb[o] = l.relu ? std::max(acc, 0.f) : acc;
      }
    }
    x.swap(y);
    in = (int)l.out;
  }
  for (int b = 0; b < B; ++b) prob[b] = 1.f / (1.f + std::exp(-x[(size_t)b * in]));
}

int main(int argc, char** argv) {
  std::string dict_path, tower_path, ids_path;
  int S = 4, dim = 8, B = 32, requests = 100;
  bool dump = false;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto val = [&]() -> const char* { if (i + 1 >= argc) { std::fprintf(stderr, "%s needs a value\n", a.c_str()); std::exit(2); } return argv[++i]; };
    if (a == "--dict") dict_path = val();
    else if (a == "--tower") tower_path = val();
    else if (a == "--ids") ids_path = val();
    else if (a == "--slots") S = std::atoi(val());
    else if (a == "--dim") dim = std::atoi(val());
    else if (a == "--batch") B = std::atoi(val());
    else if (a == "--requests") requests = std::atoi(val());
    else if (a == "--dump") dump = true;
    else { std::fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
  }
  try {
    if (dict_path.empty() || tower_path.empty() || S <= 0 || dim <= 0 || B <= 0) throw std::runtime_error("need --dict, --tower, --slots, --dim");
    Dictionary d;
    d.load(dict_path, dim);
    const std::vector<Layer> tower = load_tower(tower_path);
    if ((int)tower.front().in != S * dim) throw std::runtime_error("the tower's input width is not slots x dim");
    if (tower.back().out != 1) throw std::runtime_error("the tower's last layer must have one output");
    std::vector<float> x, y;
    if (!ids_path.empty()) {                     // one request from a file: S lines of B ids
      std::ifstream f(ids_path);
      std::vector<uint64_t> ids;
      std::string line;
      int lines = 0;
      while (std::getline(f, line) && lines < S) {
        std::istringstream ls(line);
        uint64_t v;
        size_t before = ids.size();
        while (ls >> v) ids.push_back(v);
        if (lines == 0) B = (int)(ids.size() - before);
        else if ((int)(ids.size() - before) != B) throw std::runtime_error("every line of the request needs the same number of ids");
        ++lines;
      }
      if (lines != S || B <= 0) throw std::runtime_error("the request needs one line of ids per slot");
      std::vector<float> prob(B);
      infer(d, tower, ids.data(), S, B, x, y, prob.data());
      if (dump) for (float p : prob) std::printf("%.8f\n", p);
      return 0;
    }
    std::mt19937_64 rng(0);
    std::vector<uint64_t> ids((size_t)S * B);
    std::vector<float> prob(B);
    std::vector<double> lat;
    double mean = 0;
    for (int r = 0; r < requests; ++r) {
      for (auto& v : ids) v = d.all_signs.empty() ? rng() : d.all_signs[rng() % d.all_signs.size()];
      const auto t0 = std::chrono::steady_clock::now();
      infer(d, tower, ids.data(), S, B, x, y, prob.data());
      lat.push_back(std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
      for (float p : prob) mean += p;
    }
    std::sort(lat.begin(), lat.end());
    std::printf("{\"dictionary_rows\": %zu, \"requests\": %d, \"batch\": %d, \"p50_ms\": %.4f, \"p99_ms\": %.4f, \"mean_probability\": %.6f}\n",
                d.all_signs.size(), requests, B, lat[lat.size() / 2], lat[std::max<size_t>(1, (size_t)(lat.size() * 0.99)) - 1],
                mean / ((double)requests * B));
  } catch (const std::exception& e) {
    std::fprintf(stderr, "tn_serve: %s\n", e.what());
    return 1;
  }
  return 0;
}
