// Plain C++ runtime (module _tn_cpu): the reference's parameter-server algorithms restated
// without MPI/brpc/TensorFlow, plus the checkpoint readers / writers shared by the CPU and the
// GPU tables.  It serves three purposes: the CPU execution path of the framework, the
// correctness oracle of every sm_100a kernel, and the timed CPU baseline.
//
// Restated from the reference:
//   * sparse table = 8 lock-striped hash maps per shard, rows from a fixed-size slab pool
//     (core/ps/optimizer/optimizer_kernel.h:254-437,439-560, core/utility/allocator.h:26-129)
//   * per-sign optimizer math (core/ps/optimizer/{ada_grad,adam,ftrl}_kernel.cc)
//   * on-disk formats of sparse blocks, dense shards and batch-norm tables
//     (optimizer_kernel.h:324-420,462-538, core/ps/table/dense_table.cc:103-157,
//      core/ps/table/bn_table.cc:171-214), gzip through zlib as the reference does through
//     TensorFlow's ZlibOutputBuffer (core/utility/file_io.cc:39-87)
//   * first-occurrence dedup of a batch's signs with show / click counting
//     (core/kernels/sparse_table_ops.cc:113-137,274-297)
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <zlib.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>
#include <dirent.h>
#include <sys/stat.h>

#include "tn_hash.h"

namespace py = pybind11;
using tn::kAdaGrad;
using tn::kAdam;
using tn::kFtrl;

namespace {

// ------------------------------------------------------------------------------------------
// Fixed-size slab pool: rows are carved from slabs of 65536 objects and recycled through a
// free list (the reference's Allocator<T>).
// ------------------------------------------------------------------------------------------
class RowPool {
 public:
  RowPool(size_t floats_per_row, size_t rows_per_slab = 1 << 16) : n_(floats_per_row), per_slab_(rows_per_slab) {}
  float* allocate() {
    if (!free_.empty()) { float* p = free_.back(); free_.pop_back(); return p; }
    if (used_ == per_slab_ || slabs_.empty()) {
      slabs_.emplace_back(new float[n_ * per_slab_]);
      used_ = 0;
    }
    return slabs_.back().get() + n_ * (used_++);
  }
  void deallocate(float* p) { free_.push_back(p); }
  size_t slabs() const { return slabs_.size(); }

 private:
  size_t n_, per_slab_, used_ = 0;
  std::vector<std::unique_ptr<float[]>> slabs_;
  std::vector<float*> free_;
};

struct KeyHash {
  size_t operator()(uint64_t sign) const { return std::hash<uint64_t>()((sign >> 32) | (sign << 32)); }
};

struct Block {
  std::unordered_map<uint64_t, float*, KeyHash> map;
  std::mutex mu;
  std::unique_ptr<RowPool> pool;
};

const char* opt_name(int kind) { return kind == kAdaGrad ? "AdaGrad" : kind == kAdam ? "Adam" : "Ftrl"; }

// One optimizer step on a row stored as  w | slots | counters  (layout in tn_hash.h).
void apply_row(const tn::SparseOptParams& o, float* row, const float* g, float show, float click, int dim) {
  if (o.kind == kAdaGrad) {
    row[dim + 1] += show;
    row[dim + 2] += click;
    reinterpret_cast<int32_t*>(row)[dim + 3] = 0;
    double add = 0;
    for (int i = 0; i < dim; ++i) add += (double)g[i] * g[i];
    row[dim] += (float)(add / dim);
    const float denom = o.eps + std::sqrt(row[dim]);
    for (int i = 0; i < dim; ++i) row[i] -= o.lr * g[i] / denom;
  } else if (o.kind == kAdam) {
    float* m = row + dim;
    float* v = row + 2 * dim;
    reinterpret_cast<int32_t*>(row)[3 * dim + 1] += (int)show;
    for (int i = 0; i < dim; ++i) {
      m[i] = o.beta1 * m[i] + (1 - o.beta1) * g[i];
      v[i] = o.beta2 * v[i] + (1 - o.beta2) * g[i] * g[i];
      row[i] -= o.lr * m[i] / (o.eps + std::sqrt(v[i]));
    }
  } else {
    float* z = row + dim;
    float* n = row + 2 * dim;
    reinterpret_cast<int32_t*>(row)[3 * dim + 1] += (int)show;
    for (int i = 0; i < dim; ++i) {
      float g2 = g[i] * g[i];
      z[i] += g[i] - o.lr * (std::sqrt(n[i] + g2) - std::sqrt(n[i])) * row[i];
      n[i] += g2;
      if (std::fabs(z[i]) <= o.lambda1) {
        row[i] = 0;
      } else {
        float w = -1.f / ((o.ftrl_beta + std::sqrt(n[i])) * o.lr + o.lambda2);
        row[i] = w * (z[i] > 0 ? z[i] - o.lambda1 : z[i] + o.lambda1);
      }
    }
  }
}

class CpuSparseTable {
 public:
  CpuSparseTable(py::dict opt, int dim, bool use_cvm, int shard_num, int shard_id)
      : dim_(dim), use_cvm_(use_cvm), shard_num_(shard_num), shard_id_(shard_id) {
    set_opt(opt);
    rf_ = tn::row_floats(o_.kind, dim);
    for (auto& b : blocks_) b.pool.reset(new RowPool(rf_));
  }

  void set_opt(py::dict d) {
    o_.kind = d["kind"].cast<int>(); o_.lr = d["lr"].cast<float>(); o_.eps = d["eps"].cast<float>();
    o_.beta1 = d["beta1"].cast<float>(); o_.beta2 = d["beta2"].cast<float>();
    o_.initial_g2sum = d["initial_g2sum"].cast<float>(); o_.initial_scale = d["initial_scale"].cast<float>();
    o_.ftrl_beta = d["ftrl_beta"].cast<float>(); o_.lambda1 = d["lambda1"].cast<float>(); o_.lambda2 = d["lambda2"].cast<float>();
    o_.zero_init = d["zero_init"].cast<int>(); o_.seed = d["seed"].cast<uint64_t>();
  }

  int pdim() const { return dim_ + (use_cvm_ ? 2 : 0); }

  float* find_or_create(uint64_t sign) {
    Block& b = blocks_[tn::block_of(sign)];
    std::lock_guard<std::mutex> lock(b.mu);
    auto ins = b.map.insert({sign, nullptr});
    if (ins.second) {
      float* row = b.pool->allocate();
      for (int i = 0; i < dim_; ++i) row[i] = o_.zero_init ? 0.f : tn::init_weight(o_.seed, sign, i, dim_, o_.initial_scale);
      for (int i = dim_; i < rf_; ++i) row[i] = 0.f;
      if (o_.kind == kAdaGrad) row[dim_] = o_.initial_g2sum;
      ins.first->second = row;
    }
    return ins.first->second;
  }

  // rows of weights (+ the two CVM columns) in request order; creates missing rows
  py::array_t<float> pull(py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs) {
    const ssize_t n = signs.shape(0);
    const int pd = pdim();
    py::array_t<float> out({n, (ssize_t)pd});
    const uint64_t* s = signs.data();
    float* o = out.mutable_data();
    {
      py::gil_scoped_release rel;
      for (ssize_t i = 0; i < n; ++i) {
        const float* row = find_or_create(tn::canon_key(s[i]));
        std::memcpy(o + i * pd, row, sizeof(float) * dim_);
        if (use_cvm_) {
          float show = 0, click = 0;
          if (o_.kind == kAdaGrad) { show = row[dim_ + 1]; click = row[dim_ + 2]; }
          o[i * pd + dim_] = o_.kind == kAdaGrad ? show : 0.f;
          o[i * pd + dim_ + 1] = o_.kind == kAdaGrad ? std::log(click + 1) - std::log(show + 1) : 0.f;
        }
      }
    }
    return out;
  }

  void push(py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs,
            py::array_t<float, py::array::c_style | py::array::forcecast> grads,
            py::array_t<float, py::array::c_style | py::array::forcecast> shows,
            py::array_t<float, py::array::c_style | py::array::forcecast> clicks) {
    const ssize_t n = signs.shape(0);
    if (grads.shape(0) != n || grads.shape(1) < dim_) throw std::invalid_argument("push: grads must be [n, >= dim]");
    const ssize_t gld = grads.shape(1);
    const uint64_t* s = signs.data();
    const float* g = grads.data();
    const float* sh = shows.data();
    const float* cl = clicks.data();
    py::gil_scoped_release rel;
    for (ssize_t i = 0; i < n; ++i) {
      const uint64_t sign = tn::canon_key(s[i]);
      Block& b = blocks_[tn::block_of(sign)];
      std::lock_guard<std::mutex> lock(b.mu);
      auto it = b.map.find(sign);
      if (it == b.map.end()) throw std::runtime_error("embedding of sign " + std::to_string(sign) + " not create yet, something must be wrong");
      apply_row(o_, it->second, g + i * gld, sh[i], cl[i], dim_);
    }
  }

  size_t size() const {
    size_t n = 0;
    for (auto& b : blocks_) n += b.map.size();
    return n;
  }

  void show_decay(float rate, int delta_days) {
    for (auto& b : blocks_)
      for (auto& kv : b.map) {
        float* row = kv.second;
        if (o_.kind == kAdaGrad) {
          row[dim_ + 1] *= rate; row[dim_ + 2] *= rate;
          reinterpret_cast<int32_t*>(row)[dim_ + 3] += delta_days;
        } else if (o_.kind == kFtrl) {
          row[3 * dim_] *= rate;
        }
      }
  }

  py::tuple dump() const {
    const size_t n = size();
    py::array_t<uint64_t> signs((ssize_t)n);
    py::array_t<float> rows({(ssize_t)n, (ssize_t)rf_});
    uint64_t* s = signs.mutable_data();
    float* r = rows.mutable_data();
    size_t i = 0;
    for (auto& b : blocks_)
      for (auto& kv : b.map) {
        s[i] = kv.first;
        std::memcpy(r + i * rf_, kv.second, sizeof(float) * rf_);
        ++i;
      }
    return py::make_tuple(signs, rows);
  }

  void load_rows(py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs,
                 py::array_t<float, py::array::c_style | py::array::forcecast> rows) {
    const ssize_t n = signs.shape(0);
    if (rows.shape(0) != n || rows.shape(1) != rf_) throw std::invalid_argument("load_rows: rows must be [n, row_floats]");
    const uint64_t* s = signs.data();
    const float* r = rows.data();
    for (ssize_t i = 0; i < n; ++i) {
      const uint64_t sign = tn::canon_key(s[i]);
      Block& b = blocks_[tn::block_of(sign)];
      std::lock_guard<std::mutex> lock(b.mu);
      auto ins = b.map.insert({sign, nullptr});
      if (ins.second) ins.first->second = b.pool->allocate();
      std::memcpy(ins.first->second, r + i * rf_, sizeof(float) * rf_);
    }
  }

  void clear() {
    for (auto& b : blocks_) { b.map.clear(); b.pool.reset(new RowPool(rf_)); }
  }

  int dim_, rf_;
  bool use_cvm_;
  int shard_num_, shard_id_;
  tn::SparseOptParams o_{};
  mutable Block blocks_[tn::kSparseBlockNum];
};

// ------------------------------------------------------------------------------------------
// first-occurrence dedup with show / click counting
// ------------------------------------------------------------------------------------------
py::tuple unique_first_occurrence(py::array_t<int64_t, py::array::c_style | py::array::forcecast> ids,
                                  py::object labels_obj) {
  const ssize_t n = ids.shape(0);
  const int64_t* x = ids.data();
  const float* lab = nullptr;
  py::array_t<float, py::array::c_style | py::array::forcecast> labels;
  if (!labels_obj.is_none()) {
    labels = labels_obj.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>();
    if (labels.shape(0) != n) throw std::invalid_argument("labels must have one entry per id");
    lab = labels.data();
  }
  std::unordered_map<uint64_t, int> first;
  first.reserve((size_t)n * 2);
  std::vector<uint64_t> uniq;
  std::vector<float> show, click;
  py::array_t<int32_t> inverse(n);
  int32_t* inv = inverse.mutable_data();
  for (ssize_t i = 0; i < n; ++i) {
    const uint64_t key = tn::canon_key((uint64_t)x[i]);
    auto ins = first.insert({key, (int)uniq.size()});
    if (ins.second) { uniq.push_back(key); show.push_back(0.f); click.push_back(0.f); }
    const int v = ins.first->second;
    inv[i] = v;
    show[v] += 1.f;
    if (lab) click[v] += lab[i];
  }
  py::array_t<uint64_t> u((ssize_t)uniq.size());
  py::array_t<float> s((ssize_t)uniq.size()), c((ssize_t)uniq.size());
  std::memcpy(u.mutable_data(), uniq.data(), uniq.size() * 8);
  std::memcpy(s.mutable_data(), show.data(), show.size() * 4);
  std::memcpy(c.mutable_data(), click.data(), click.size() * 4);
  return py::make_tuple(u, inverse, s, c);
}

// ------------------------------------------------------------------------------------------
// gzip helpers
// ------------------------------------------------------------------------------------------
void mkdirs(const std::string& dir) {
  std::string cur;
  for (size_t i = 0; i < dir.size(); ++i) {
    cur.push_back(dir[i]);
    if (dir[i] == '/' || i + 1 == dir.size()) ::mkdir(cur.c_str(), 0777);
  }
}

class GzWriter {
 public:
  explicit GzWriter(const std::string& path) {
    f_ = gzopen(path.c_str(), "wb6");
    if (!f_) throw std::runtime_error("cannot open for writing: " + path);
    gzbuffer(f_, 1 << 20);
  }
  ~GzWriter() { if (f_) gzclose(f_); }
  void write(const void* p, size_t n) {
    if (n && gzwrite(f_, p, (unsigned)n) != (int)n) throw std::runtime_error("gzwrite failed");
  }
  void write(const std::string& s) { write(s.data(), s.size()); }

 private:
  gzFile f_;
};

std::string gz_read_all(const std::string& path) {
  gzFile f = gzopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("cannot open for reading: " + path);
  gzbuffer(f, 1 << 20);
  std::string out;
  std::vector<char> buf(1 << 20);
  int n;
  while ((n = gzread(f, buf.data(), (unsigned)buf.size())) > 0) out.append(buf.data(), (size_t)n);
  gzclose(f);
  if (n < 0) throw std::runtime_error("gzread failed: " + path);
  return out;
}

inline void append_g(std::string& s, float v) {   // what `ostream << float` prints: %g, 6 significant digits
  char b[32];
  int n = std::snprintf(b, sizeof b, "%g", (double)v);
  s.append(b, (size_t)n);
}

struct EvictRule {   // DeleteByShow, applied only while saving
  bool enabled = false;
  float show_threshold = 0;
  int no_show_days = 1000;
  int logic = 0;
  bool drop(int kind, const float* row, int dim) const {
    if (!enabled) return false;
    if (kind == kAdaGrad) {
      const float show = row[dim + 1];
      const int nsd = reinterpret_cast<const int32_t*>(row)[dim + 3];
      return logic == 1 ? (show < show_threshold && nsd > no_show_days) : (show < show_threshold || nsd > no_show_days);
    }
    if (kind == kFtrl) return row[3 * dim] < show_threshold;
    return false;
  }
};

// rows are in table layout ([w|g2sum|show|click|no_show_days] or [w|s1|s2|show|delta_show])
void block_header(std::string& buf, bool bin, int kind, int dim) {
  if (bin) {
    int32_t d = dim;
    buf.append(reinterpret_cast<const char*>(&d), 4);
  } else {
    buf += "opt_name:"; buf += opt_name(kind); buf += "\n";
    buf += "dim:" + std::to_string(dim) + "\n";
  }
}

// Appends one record; returns false when the eviction rule drops the row.
inline bool append_record(std::string& buf, bool bin, int kind, int dim, bool use_cvm, uint64_t sign, const float* row,
                          const EvictRule& rule) {
  if (rule.drop(kind, row, dim)) return false;
  if (bin) {
    buf.append(reinterpret_cast<const char*>(&sign), 8);
    if (kind == kAdaGrad) {
      buf.append(reinterpret_cast<const char*>(row), 4 * dim);          // w
      buf.append(reinterpret_cast<const char*>(row + dim), 4);          // g2sum
      buf.append(reinterpret_cast<const char*>(row + dim + 1), 4);      // show
      buf.append(reinterpret_cast<const char*>(row + dim + 3), 4);      // no_show_days (int32)
      if (use_cvm) buf.append(reinterpret_cast<const char*>(row + dim + 2), 4);  // click
    } else {
      buf.append(reinterpret_cast<const char*>(row), 4 * 3 * dim);      // w, m|z, v|n
      buf.append(reinterpret_cast<const char*>(row + 3 * dim), 4);      // show
    }
  } else {
    buf += std::to_string(sign); buf += "\t";
    if (kind == kAdaGrad) {
      buf += std::to_string(dim); buf += "\t";
      for (int k = 0; k < dim; ++k) { append_g(buf, row[k]); buf += "\t"; }
      append_g(buf, row[dim]); buf += "\t";
      append_g(buf, row[dim + 1]); buf += "\t";
      buf += std::to_string(reinterpret_cast<const int32_t*>(row)[dim + 3]); buf += "\t";
      if (use_cvm) append_g(buf, row[dim + 2]);
    } else {
      for (int k = 0; k < dim; ++k) {
        append_g(buf, row[k]); buf += "\t";
        append_g(buf, row[dim + k]); buf += "\t";
        append_g(buf, row[2 * dim + k]); buf += "\t";
      }
      append_g(buf, row[3 * dim]);
    }
    buf += "\n";
  }
  return true;
}

// Streaming writer of one rank directory: the eight block files stay open while the table arrives in chunks,
// so a shard far larger than host memory can be saved.  Every append serialises and compresses the eight
// blocks on eight threads (the reference saves with one thread per block as well,
// core/ps/optimizer/optimizer_kernel.h:462-486).
class SparseDirWriter {
 public:
  SparseDirWriter(const std::string& dir, const std::string& mode, int kind, int dim, bool use_cvm, bool evict,
                  float show_threshold, int no_show_days, int logic)
      : bin_(mode == "bin"), kind_(kind), dim_(dim), use_cvm_(use_cvm), rf_(tn::row_floats(kind, dim)),
        rule_{evict, show_threshold, no_show_days, logic} {
    mkdirs(dir);
    for (int b = 0; b < tn::kSparseBlockNum; ++b) {
      // text blocks keep the reference's file name; binary blocks carry the `_bin` suffix its reader
      // needs to recognise them (core/ps/optimizer/optimizer_kernel.h:488-517)
      w_.emplace_back(new GzWriter(dir + "/block_" + std::to_string(b) + (bin_ ? "_bin" : "") + ".gz"));
      std::string h;
      block_header(h, bin_, kind_, dim_);
      w_[b]->write(h);
    }
  }

  // records [offsets[b], offsets[b+1]) belong to block b (what the device-side export produces)
  void append_grouped(py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs,
                      py::array_t<float, py::array::c_style | py::array::forcecast> rows,
                      py::array_t<int64_t, py::array::c_style | py::array::forcecast> offsets) {
    check_open();
    const ssize_t n = signs.shape(0);
    if (rows.shape(0) != n || (n > 0 && rows.shape(1) != rf_)) throw std::invalid_argument("append: rows must be [n, row_floats]");
    if (offsets.shape(0) != tn::kSparseBlockNum + 1) throw std::invalid_argument("append_grouped: offsets must have 9 entries");
    const int64_t* off = offsets.data();
    if (off[0] != 0 || off[tn::kSparseBlockNum] != n) throw std::invalid_argument("append_grouped: offsets do not cover the records");
    const uint64_t* s = signs.data();
    const float* r = rows.data();
    run_blocks([&](int b, std::string& buf) {
      int64_t kept = 0;
      for (int64_t i = off[b]; i < off[b + 1]; ++i) {
        if (tn::block_of(s[i]) != b) throw std::runtime_error("append_grouped: record outside its block range");
        kept += append_record(buf, bin_, kind_, dim_, use_cvm_, s[i], r + (size_t)i * rf_, rule_);
        if (buf.size() > (1 << 20)) { w_[b]->write(buf); buf.clear(); }
      }
      return kept;
    });
  }

  // records in any order
  void append(py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs,
              py::array_t<float, py::array::c_style | py::array::forcecast> rows) {
    check_open();
    const ssize_t n = signs.shape(0);
    if (rows.shape(0) != n || (n > 0 && rows.shape(1) != rf_)) throw std::invalid_argument("append: rows must be [n, row_floats]");
    const uint64_t* s = signs.data();
    const float* r = rows.data();
    std::vector<std::vector<size_t>> per(tn::kSparseBlockNum);
    for (ssize_t i = 0; i < n; ++i) per[tn::block_of(s[i])].push_back((size_t)i);
    run_blocks([&](int b, std::string& buf) {
      int64_t kept = 0;
      for (size_t i : per[b]) {
        kept += append_record(buf, bin_, kind_, dim_, use_cvm_, s[i], r + i * rf_, rule_);
        if (buf.size() > (1 << 20)) { w_[b]->write(buf); buf.clear(); }
      }
      return kept;
    });
  }

  int64_t close() {
    if (!closed_) {
      for (auto& w : w_) { w->write(std::string("\n")); w.reset(); }   // the `<< std::endl` after the block
      closed_ = true;
    }
    return written_;
  }

 private:
  void check_open() const { if (closed_) throw std::runtime_error("SparseDirWriter is closed"); }
  template <class F>
  void run_blocks(F fn) {
    std::vector<std::thread> threads;
    std::vector<std::string> errors(tn::kSparseBlockNum);
    std::vector<int64_t> kept(tn::kSparseBlockNum, 0);
    {
      py::gil_scoped_release rel;
      for (int b = 0; b < tn::kSparseBlockNum; ++b) {
        threads.emplace_back([&, b]() {
          try {
            std::string buf;
            buf.reserve(1 << 20);
            kept[b] = fn(b, buf);
            w_[b]->write(buf);
          } catch (const std::exception& e) { errors[b] = e.what(); }
        });
      }
      for (auto& t : threads) t.join();
    }
    for (auto& e : errors) if (!e.empty()) throw std::runtime_error(e);
    for (int64_t k : kept) written_ += k;
  }

  bool bin_;
  int kind_, dim_;
  bool use_cvm_;
  int rf_;
  EvictRule rule_;
  std::vector<std::unique_ptr<GzWriter>> w_;
  bool closed_ = false;
  int64_t written_ = 0;
};

int write_sparse_dir(const std::string& dir, const std::string& mode, int kind, int dim, bool use_cvm,
                     py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs,
                     py::array_t<float, py::array::c_style | py::array::forcecast> rows, bool evict, float show_threshold,
                     int no_show_days, int logic) {
  SparseDirWriter w(dir, mode, kind, dim, use_cvm, evict, show_threshold, no_show_days, logic);
  w.append(signs, rows);
  w.close();
  return (int)signs.shape(0);
}

std::vector<std::string> list_dir(const std::string& dir) {
  std::vector<std::string> out;
  DIR* d = opendir(dir.c_str());
  if (!d) return out;
  while (dirent* e = readdir(d)) {
    std::string n = e->d_name;
    if (n != "." && n != "..") out.push_back(n);
  }
  closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}

struct ParsedBlock {
  std::vector<uint64_t> signs;
  std::vector<float> rows;
};

// One text data line -> one row appended to `out` (empty lines are skipped).  `line` is modified in place.
void parse_txt_line(std::string& line, int kind, int dim, bool use_cvm, std::vector<const char*>& tok, ParsedBlock& out) {
  const int rf = tn::row_floats(kind, dim);
  tok.clear();
  char* p = &line[0];
  while (*p) {
    while (*p == '\t' || *p == ' ' || *p == '\r') ++p;
    if (!*p) break;
    tok.push_back(p);
    while (*p && *p != '\t' && *p != ' ' && *p != '\r') ++p;
    if (*p) *p++ = 0;
  }
  if (tok.empty()) return;
  const uint64_t sign = std::strtoull(tok[0], nullptr, 10);
  out.signs.push_back(sign);
  const size_t base = out.rows.size();
  out.rows.resize(base + rf, 0.f);
  float* row = out.rows.data() + base;
  if (kind == kAdaGrad) {
    // sign dim w*dim g2sum show [no_show_days [click]]; files written before no_show_days existed have dim+4 columns
    const int nt = (int)tok.size();
    if (nt < dim + 4) throw std::runtime_error("sparse block: short AdaGrad line");
    for (int k = 0; k < dim; ++k) row[k] = std::strtof(tok[2 + k], nullptr);
    row[dim] = std::strtof(tok[2 + dim], nullptr);
    row[dim + 1] = std::strtof(tok[3 + dim], nullptr);
    if (nt >= dim + 5) reinterpret_cast<int32_t*>(row)[dim + 3] = std::atoi(tok[4 + dim]);
    if (nt >= dim + 6 && use_cvm) row[dim + 2] = std::strtof(tok[5 + dim], nullptr);
  } else {
    if ((int)tok.size() < 3 * dim + 2) throw std::runtime_error("sparse block: short Adam/Ftrl line");
    for (int k = 0; k < dim; ++k) {
      row[k] = std::strtof(tok[1 + 3 * k], nullptr);
      row[dim + k] = std::strtof(tok[2 + 3 * k], nullptr);
      row[2 * dim + k] = std::strtof(tok[3 + 3 * k], nullptr);
    }
    row[3 * dim] = std::strtof(tok[1 + 3 * dim], nullptr);
  }
}

void check_txt_header(const std::string& l1, const std::string& l2, int dim, const std::string& want_opt) {
  if (l1.rfind("opt_name:", 0) != 0) throw std::runtime_error("sparse block: missing opt_name header");
  const std::string name = l1.substr(9);
  if (name != want_opt)
    throw std::runtime_error("last trained model with optimizer is:" + name + " but current model use:" + want_opt +
                             " instead. you must make sure that use same optimizer when incremental training");
  if (l2.rfind("dim:", 0) != 0) throw std::runtime_error("sparse block: missing dim header");
  const int fdim = std::atoi(l2.c_str() + 4);
  if (fdim != dim) throw std::runtime_error("sparse block: dim " + std::to_string(fdim) + " != table dim " + std::to_string(dim));
}

size_t bin_record_bytes(int kind, int dim, bool use_cvm) {
  return 8 + (kind == kAdaGrad ? 4 * (size_t)(dim + 3 + (use_cvm ? 1 : 0)) : 4 * (size_t)(3 * dim + 1));
}

// One binary record at `p` -> one row appended to `out`.
void parse_bin_record(const char* rec, int kind, int dim, bool use_cvm, ParsedBlock& out) {
  const int rf = tn::row_floats(kind, dim);
  uint64_t sign;
  std::memcpy(&sign, rec, 8);
  const char* p = rec + 8;
  out.signs.push_back(sign);
  const size_t base = out.rows.size();
  out.rows.resize(base + rf, 0.f);
  float* row = out.rows.data() + base;
  if (kind == kAdaGrad) {
    std::memcpy(row, p, 4 * dim);
    std::memcpy(row + dim, p + 4 * dim, 4);           // g2sum
    std::memcpy(row + dim + 1, p + 4 * dim + 4, 4);   // show
    std::memcpy(row + dim + 3, p + 4 * dim + 8, 4);   // no_show_days
    if (use_cvm) std::memcpy(row + dim + 2, p + 4 * dim + 12, 4);
  } else {
    std::memcpy(row, p, 4 * 3 * dim);
    std::memcpy(row + 3 * dim, p + 4 * 3 * dim, 4);
  }
}

void parse_txt_block(const std::string& data, int kind, int dim, bool use_cvm, const std::string& want_opt, ParsedBlock& out) {
  size_t pos = 0;
  auto next_line = [&](std::string& line) -> bool {
    if (pos >= data.size()) return false;
    size_t e = data.find('\n', pos);
    if (e == std::string::npos) e = data.size();
    line.assign(data, pos, e - pos);
    pos = e + 1;
    return true;
  };
  std::string l1, l2, line;
  if (!next_line(l1)) throw std::runtime_error("sparse block: missing opt_name header");
  if (!next_line(l2)) throw std::runtime_error("sparse block: missing dim header");
  check_txt_header(l1, l2, dim, want_opt);
  std::vector<const char*> tok;
  while (next_line(line)) {
    if (!line.empty()) parse_txt_line(line, kind, dim, use_cvm, tok, out);
  }
}

void parse_bin_block(const std::string& data, int kind, int dim, bool use_cvm, ParsedBlock& out) {
  if (data.size() < 4) throw std::runtime_error("sparse block: truncated binary header");
  int32_t fdim;
  std::memcpy(&fdim, data.data(), 4);
  if (fdim != dim) throw std::runtime_error("sparse block: dim " + std::to_string(fdim) + " != table dim " + std::to_string(dim));
  const size_t rec = bin_record_bytes(kind, dim, use_cvm);
  for (size_t pos = 4; pos + rec <= data.size(); pos += rec) parse_bin_record(data.data() + pos, kind, dim, use_cvm, out);
}

// name = <prefix><digits><suffix>.gz  (the reference matches `(.*?)(\d+)(.*)\.gz`); returns false for other names
bool split_block_name(const std::string& f, std::string* suffix) {
  if (f.size() < 4 || f.compare(f.size() - 3, 3, ".gz") != 0) return false;
  const std::string stem = f.substr(0, f.size() - 3);
  size_t d0 = 0;
  while (d0 < stem.size() && !(stem[d0] >= '0' && stem[d0] <= '9')) ++d0;
  if (d0 == stem.size()) return false;
  size_t d1 = d0;
  while (d1 < stem.size() && stem[d1] >= '0' && stem[d1] <= '9') ++d1;
  *suffix = stem.substr(d1);
  return true;
}

// Streams ONE block file: every call to next() decompresses and parses up to `max_rows` further rows, so the
// host never holds more than one piece of a block however large the file is.  The reference parses a block as a
// stream as well, row by row (core/ps/optimizer/optimizer_kernel.h:366-420).  Mode: an explicit `_bin` / `_txt`
// suffix decides, otherwise the first bytes are sniffed (`opt_name:` => text).
class SparseBlockReader {
 public:
  SparseBlockReader(const std::string& path, int kind, int dim, bool use_cvm)
      : path_(path), kind_(kind), dim_(dim), use_cvm_(use_cvm), rf_(tn::row_floats(kind, dim)) {
    f_ = gzopen(path.c_str(), "rb");
    if (!f_) throw std::runtime_error("cannot open for reading: " + path);
    gzbuffer(f_, 1 << 20);
    std::string name = path.substr(path.find_last_of('/') == std::string::npos ? 0 : path.find_last_of('/') + 1), suffix;
    split_block_name(name, &suffix);
    fill();
    if (suffix == "_bin") bin_ = true;
    else if (suffix == "_txt") bin_ = false;
    else bin_ = buf_.compare(0, 9, "opt_name:") != 0;
    if (bin_) {
      while (buf_.size() < 4 && !eof_) fill();
      if (buf_.size() < 4) throw std::runtime_error("sparse block: truncated binary header");
      int32_t fdim;
      std::memcpy(&fdim, buf_.data(), 4);
      if (fdim != dim) throw std::runtime_error("sparse block: dim " + std::to_string(fdim) + " != table dim " + std::to_string(dim));
      pos_ = 4;
    } else {
      std::string l1, l2;
      if (!take_line(l1)) throw std::runtime_error("sparse block: missing opt_name header");
      if (!take_line(l2)) throw std::runtime_error("sparse block: missing dim header");
      check_txt_header(l1, l2, dim, opt_name(kind));
    }
  }
  ~SparseBlockReader() { if (f_) gzclose(f_); }

  // (signs uint64 [m], rows float32 [m, row_floats]) with m <= max_rows; m == 0 only at the end of the file
  py::tuple next(int64_t max_rows) {
    ParsedBlock out;
    {
      py::gil_scoped_release rel;
      out.signs.reserve((size_t)std::min<int64_t>(max_rows, 1 << 20));
      if (bin_) {
        const size_t rec = bin_record_bytes(kind_, dim_, use_cvm_);
        while ((int64_t)out.signs.size() < max_rows) {
          while (buf_.size() - pos_ < rec && !eof_) fill();
          if (buf_.size() - pos_ < rec) break;          // the trailing newline byte (or nothing) is left
          parse_bin_record(buf_.data() + pos_, kind_, dim_, use_cvm_, out);
          pos_ += rec;
        }
      } else {
        std::string line;
        std::vector<const char*> tok;
        while ((int64_t)out.signs.size() < max_rows && take_line(line)) {
          if (!line.empty()) parse_txt_line(line, kind_, dim_, use_cvm_, tok, out);
        }
      }
    }
    const ssize_t n = (ssize_t)out.signs.size();
    py::array_t<uint64_t> signs(n);
    py::array_t<float> rows({n, (ssize_t)rf_});
    if (n) {
      std::memcpy(signs.mutable_data(), out.signs.data(), (size_t)n * 8);
      std::memcpy(rows.mutable_data(), out.rows.data(), (size_t)n * rf_ * 4);
    }
    return py::make_tuple(signs, rows);
  }
  bool is_binary() const { return bin_; }

 private:
  void fill() {      // drop what has been consumed, read another piece
    if (pos_ > 0) { buf_.erase(0, pos_); pos_ = 0; }
    const size_t old = buf_.size();
    buf_.resize(old + (1 << 20));
    const int n = gzread(f_, &buf_[old], 1 << 20);
    if (n < 0) throw std::runtime_error("gzread failed: " + path_);
    buf_.resize(old + (size_t)n);
    if (n == 0) eof_ = true;
  }
  bool take_line(std::string& line) {
    for (;;) {
      const size_t e = buf_.find('\n', pos_);
      if (e != std::string::npos) { line.assign(buf_, pos_, e - pos_); pos_ = e + 1; return true; }
      if (eof_) {
        if (pos_ >= buf_.size()) return false;
        line.assign(buf_, pos_, buf_.size() - pos_);
        pos_ = buf_.size();
        return true;
      }
      fill();
    }
  }
  std::string path_;
  int kind_, dim_;
  bool use_cvm_;
  int rf_;
  gzFile f_ = nullptr;
  std::string buf_;
  size_t pos_ = 0;
  bool eof_ = false, bin_ = false;
};

// Block files of a rank directory (names the reference's reader would accept), sorted.
std::vector<std::string> list_block_files(const std::string& dir) {
  std::vector<std::string> out;
  for (auto& f : list_dir(dir)) {
    std::string suf;
    if (split_block_name(f, &suf)) out.push_back(f);
  }
  std::sort(out.begin(), out.end());
  return out;
}

// `sign \t [ \t w0 \t ... \t ]` lines of an exported embedding dictionary (brackets optional), streamed like a block.
class DictionaryReader {
 public:
  explicit DictionaryReader(const std::string& path) : path_(path) {
    f_ = gzopen(path.c_str(), "rb");      // reads plain files as well
    if (!f_) throw std::runtime_error("cannot open for reading: " + path);
    gzbuffer(f_, 1 << 20);
  }
  ~DictionaryReader() { if (f_) gzclose(f_); }
  // (signs uint64 [m], weights float32 [m, dim]); dim is taken from the first line; m == 0 at the end
  py::tuple next(int64_t max_rows) {
    std::vector<uint64_t> signs;
    std::vector<float> w;
    {
      py::gil_scoped_release rel;
      std::string line;
      std::vector<float> vals;
      while ((int64_t)signs.size() < max_rows && take_line(line)) {
        char* p = &line[0];
        while (*p == ' ' || *p == '\t') ++p;
        if (!*p) continue;
        char* end = nullptr;
        const uint64_t sign = std::strtoull(p, &end, 10);
        if (end == p) throw std::runtime_error("dictionary: line does not start with a sign: " + path_);
        p = end;
        vals.clear();
        while (*p) {
          while (*p == ' ' || *p == '\t' || *p == '[' || *p == ']' || *p == ',' || *p == '\r') ++p;
          if (!*p) break;
          const float v = std::strtof(p, &end);
          if (end == p) throw std::runtime_error("dictionary: bad number: " + path_);
          vals.push_back(v);
          p = end;
        }
        if (dim_ < 0) dim_ = (int)vals.size();
        if ((int)vals.size() != dim_) throw std::runtime_error("dictionary: rows of different width: " + path_);
        signs.push_back(sign);
        w.insert(w.end(), vals.begin(), vals.end());
      }
    }
    const ssize_t n = (ssize_t)signs.size();
    py::array_t<uint64_t> s(n);
    py::array_t<float> r({n, (ssize_t)std::max(dim_, 0)});
    if (n) {
      std::memcpy(s.mutable_data(), signs.data(), (size_t)n * 8);
      std::memcpy(r.mutable_data(), w.data(), w.size() * 4);
    }
    return py::make_tuple(s, r);
  }

 private:
  bool take_line(std::string& line) {
    for (;;) {
      const size_t e = buf_.find('\n', pos_);
      if (e != std::string::npos) { line.assign(buf_, pos_, e - pos_); pos_ = e + 1; return true; }
      if (eof_) {
        if (pos_ >= buf_.size()) return false;
        line.assign(buf_, pos_, buf_.size() - pos_);
        pos_ = buf_.size();
        return true;
      }
      if (pos_ > 0) { buf_.erase(0, pos_); pos_ = 0; }
      const size_t old = buf_.size();
      buf_.resize(old + (1 << 20));
      const int n = gzread(f_, &buf_[old], 1 << 20);
      if (n < 0) throw std::runtime_error("gzread failed: " + path_);
      buf_.resize(old + (size_t)n);
      if (n == 0) eof_ = true;
    }
  }
  std::string path_;
  gzFile f_ = nullptr;
  std::string buf_;
  size_t pos_ = 0;
  bool eof_ = false;
  int dim_ = -1;
};

// Reads every block file of a rank directory.  File-name rules of the reference's reader:
// `<prefix><n><suffix>.gz`; an explicit `_bin` / `_txt` suffix decides the mode, otherwise the first
// bytes are sniffed (`opt_name:` => text) so that suffix-less binary files are still read correctly.
py::tuple read_sparse_dir(const std::string& dir, int kind, int dim, bool use_cvm) {
  std::vector<std::string> files, suffixes;
  for (auto& f : list_dir(dir)) {
    std::string suf;
    if (split_block_name(f, &suf)) { files.push_back(f); suffixes.push_back(suf); }
  }
  std::vector<ParsedBlock> parsed(files.size());
  std::vector<std::string> errors(files.size());
  const std::string want = opt_name(kind);
  {
    py::gil_scoped_release rel;
    std::vector<std::thread> threads;
    for (size_t i = 0; i < files.size(); ++i) {
      threads.emplace_back([&, i]() {
        try {
          const std::string& suffix = suffixes[i];
          std::string data = gz_read_all(dir + "/" + files[i]);
          bool bin;
          if (suffix == "_bin") bin = true;
          else if (suffix == "_txt") bin = false;
          else bin = data.rfind("opt_name:", 0) != 0;
          if (bin) parse_bin_block(data, kind, dim, use_cvm, parsed[i]);
          else parse_txt_block(data, kind, dim, use_cvm, want, parsed[i]);
        } catch (const std::exception& e) { errors[i] = files[i] + ": " + e.what(); }
      });
    }
    for (auto& t : threads) t.join();
  }
  for (auto& e : errors) if (!e.empty()) throw std::runtime_error(e);
  size_t n = 0;
  for (auto& p : parsed) n += p.signs.size();
  const int rf = tn::row_floats(kind, dim);
  py::array_t<uint64_t> signs((ssize_t)n);
  py::array_t<float> rows({(ssize_t)n, (ssize_t)rf});
  size_t off = 0;
  for (auto& p : parsed) {
    std::memcpy(signs.mutable_data() + off, p.signs.data(), p.signs.size() * 8);
    std::memcpy(rows.mutable_data() + off * rf, p.rows.data(), p.rows.size() * 4);
    off += p.signs.size();
  }
  return py::make_tuple(signs, rows);
}

// ------------------------------------------------------------------------------------------
// dense shard file: plain text, 8 blocks of ceil(len/8) elements (optimizer_kernel.h:176-187)
// ------------------------------------------------------------------------------------------
void write_dense_file(const std::string& path, long long total_elements, int rank_num, int kind,
                      py::array_t<float, py::array::c_style | py::array::forcecast> w,
                      py::array_t<float, py::array::c_style | py::array::forcecast> s0,
                      py::array_t<float, py::array::c_style | py::array::forcecast> s1, py::object s2_obj, float b1p, float b2p) {
  const size_t len = (size_t)w.shape(0);
  const float* W = w.data(); const float* S0 = s0.data(); const float* S1 = s1.data();
  py::array_t<float, py::array::c_style | py::array::forcecast> s2;
  const float* S2 = nullptr;
  if (!s2_obj.is_none()) { s2 = s2_obj.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>(); S2 = s2.data(); }
  size_t slash = path.find_last_of('/');
  if (slash != std::string::npos) mkdirs(path.substr(0, slash));
  FILE* f = std::fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("cannot open for writing: " + path);
  std::string buf;
  buf += "total_elements:" + std::to_string(total_elements) + "\n";
  buf += "rank_num:" + std::to_string(rank_num) + "\n";
  const size_t per = (len + 7) / 8;
  for (size_t off = 0; off < len; off += per) {
    const size_t n = std::min(per, len - off);
    buf += std::string("opt_name:") + (kind == kAdam ? "Adam" : "AdaGrad") + "\n";
    buf += "array_size:" + std::to_string(n) + "\n";
    if (kind == kAdam) {
      buf += "beta1_power:"; append_g(buf, b1p); buf += "\n";
      buf += "beta2_power:"; append_g(buf, b2p); buf += "\n";
      for (size_t i = off; i < off + n; ++i) {
        append_g(buf, W[i]); buf += "\t"; append_g(buf, S0[i]); buf += "\t"; append_g(buf, S1[i]); buf += "\n";
      }
    } else {
      for (size_t i = off; i < off + n; ++i) {   // w d2sum g2sum m
        append_g(buf, W[i]); buf += "\t"; append_g(buf, S0[i]); buf += "\t"; append_g(buf, S1[i]); buf += "\t";
        append_g(buf, S2 ? S2[i] : 0.f); buf += "\n";
      }
    }
    buf += "\n\n";
    if (buf.size() > (1 << 22)) { std::fwrite(buf.data(), 1, buf.size(), f); buf.clear(); }
  }
  std::fwrite(buf.data(), 1, buf.size(), f);
  std::fclose(f);
}

py::dict read_dense_file(const std::string& path, int kind) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("cannot open for reading: " + path);
  std::string data;
  char tmp[1 << 16];
  size_t n;
  while ((n = std::fread(tmp, 1, sizeof tmp, f)) > 0) data.append(tmp, n);
  std::fclose(f);
  const char* p = data.c_str();
  auto after_colon = [&]() -> const char* {
    const char* c = std::strchr(p, ':');
    if (!c) throw std::runtime_error("dense file: unexpected end");
    p = c + 1;
    return p;
  };
  long long total = std::strtoll(after_colon(), const_cast<char**>(&p), 10);
  int rank_num = (int)std::strtol(after_colon(), const_cast<char**>(&p), 10);
  std::vector<float> W, S0, S1, S2;
  float b1p = 1, b2p = 1;
  const std::string want = kind == kAdam ? "Adam" : "AdaGrad";
  while (true) {
    const char* c = std::strstr(p, "opt_name:");
    if (!c) break;
    p = c + 9;
    const char* e = p;
    while (*e && *e != '\n' && *e != '\r') ++e;
    std::string name(p, e);
    if (name != want)
      throw std::runtime_error("last trained model with optimizer is:" + name + " but current model use:" + want + " instead.");
    p = e;
    long cnt = std::strtol(after_colon(), const_cast<char**>(&p), 10);
    if (kind == kAdam) {
      b1p = std::strtof(after_colon(), const_cast<char**>(&p));
      b2p = std::strtof(after_colon(), const_cast<char**>(&p));
    }
    for (long i = 0; i < cnt; ++i) {
      W.push_back(std::strtof(p, const_cast<char**>(&p)));
      S0.push_back(std::strtof(p, const_cast<char**>(&p)));
      S1.push_back(std::strtof(p, const_cast<char**>(&p)));
      if (kind != kAdam) S2.push_back(std::strtof(p, const_cast<char**>(&p)));
    }
  }
  auto to_np = [](const std::vector<float>& v) {
    py::array_t<float> a((ssize_t)v.size());
    std::memcpy(a.mutable_data(), v.data(), v.size() * 4);
    return a;
  };
  py::dict d;
  d["total_elements"] = total; d["rank_num"] = rank_num;
  d["w"] = to_np(W); d["s0"] = to_np(S0); d["s1"] = to_np(S1); d["s2"] = to_np(S2);
  d["beta1_power"] = b1p; d["beta2_power"] = b2p;
  return d;
}

// ------------------------------------------------------------------------------------------
// batch-norm table file: gzip( bool use_pctr_dnn_bn, uint32 bn_size, then per feature
// double sum, double squared_sum, double count )
// ------------------------------------------------------------------------------------------
void write_bn_file(const std::string& path, bool pctr, py::array_t<double, py::array::c_style | py::array::forcecast> sum,
                   py::array_t<double, py::array::c_style | py::array::forcecast> sq,
                   py::array_t<double, py::array::c_style | py::array::forcecast> cnt) {
  size_t slash = path.find_last_of('/');
  if (slash != std::string::npos) mkdirs(path.substr(0, slash));
  GzWriter w(path);
  const uint32_t n = (uint32_t)sum.shape(0);
  const char flag = pctr ? 1 : 0;
  w.write(&flag, 1);
  w.write(&n, 4);
  for (uint32_t i = 0; i < n; ++i) {
    w.write(sum.data() + i, 8); w.write(sq.data() + i, 8); w.write(cnt.data() + i, 8);
  }
}

py::tuple read_bn_file(const std::string& path) {
  std::string d = gz_read_all(path);
  if (d.size() < 5) throw std::runtime_error("bn table file too short: " + path);
  const bool pctr = d[0] != 0;
  uint32_t n;
  std::memcpy(&n, d.data() + 1, 4);
  if (d.size() < 5 + (size_t)n * 24) throw std::runtime_error("bn table file truncated: " + path);
  py::array_t<double> sum((ssize_t)n), sq((ssize_t)n), cnt((ssize_t)n);
  for (uint32_t i = 0; i < n; ++i) {
    std::memcpy(sum.mutable_data() + i, d.data() + 5 + (size_t)i * 24, 8);
    std::memcpy(sq.mutable_data() + i, d.data() + 5 + (size_t)i * 24 + 8, 8);
    std::memcpy(cnt.mutable_data() + i, d.data() + 5 + (size_t)i * 24 + 16, 8);
  }
  return py::make_tuple(pctr, sum, sq, cnt);
}

py::array_t<float> init_weights(uint64_t seed, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> signs, int dim,
                                float scale) {
  const ssize_t n = signs.shape(0);
  py::array_t<float> out({n, (ssize_t)dim});
  for (ssize_t i = 0; i < n; ++i)
    for (int k = 0; k < dim; ++k) out.mutable_data()[i * dim + k] = tn::init_weight(seed, tn::canon_key(signs.data()[i]), k, dim, scale);
  return out;
}

}  // namespace

#ifndef TORCH_EXTENSION_NAME
#define TORCH_EXTENSION_NAME _tn_cpu
#endif

// One dense optimizer step over a flat fp32 array in a single pass (the CPU path's counterpart of the fused dense
// kernel): Adam as in core/ps/optimizer/adam_kernel.cc:46-55 (alpha carries both beta powers, no bias correction of
// the moments themselves), AdaGrad with decayed statistics and momentum as in ada_grad_kernel.cc:42-48.  The
// gradient is zeroed on the way.  All arrays are contiguous float32 numpy views of the table's tensors.
void dense_step(int kind, py::array_t<float> w_, py::array_t<float> g_, py::array_t<float> s0_, py::array_t<float> s1_,
                py::array_t<float> s2_, double lr, double alpha, double beta1, double beta2, double eps,
                double grad_decay, double mom_decay) {
  float* w = w_.mutable_data();
  float* g = g_.mutable_data();
  float* s0 = s0_.mutable_data();
  float* s1 = s1_.mutable_data();
  float* s2 = s2_.size() ? s2_.mutable_data() : nullptr;
  const ssize_t n = w_.size();
  if (g_.size() != n || s0_.size() != n || s1_.size() != n) throw std::runtime_error("dense_step: array sizes differ");
  py::gil_scoped_release rel;
  if (kind == tn::kAdam) {
    const float a = (float)alpha, b1 = (float)beta1, b2 = (float)beta2, e = (float)eps;
    for (ssize_t i = 0; i < n; ++i) {
      const float x = g[i];
      const float m = s0[i] + (x - s0[i]) * (1.f - b1);
      const float v = s1[i] + (x * x - s1[i]) * (1.f - b2);
      s0[i] = m;
      s1[i] = v;
      w[i] -= m * a / (std::sqrt(v) + e);
      g[i] = 0.f;
    }
  } else {
    if (!s2 || s2_.size() != n) throw std::runtime_error("dense_step: AdaGrad needs the momentum array");
    const float gd = (float)grad_decay, md = (float)mom_decay, l = (float)lr, e = (float)eps;
    for (ssize_t i = 0; i < n; ++i) {
      const float x = g[i];
      const float c = s0[i] * gd + 1.f;
      const float q = s1[i] * gd + x * x;
      const float m = s2[i] + (x - s2[i]) * (1.f - md);
      s0[i] = c;
      s1[i] = q;
      s2[i] = m;
      w[i] -= l * m / (std::sqrt(q) / std::sqrt(c) + e);
      g[i] = 0.f;
    }
  }
}

void bind_tfrecord(py::module_& m);   // tfrecord.cpp: TFRecord / tf.train.Example input pipeline

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  bind_tfrecord(m);
  py::class_<CpuSparseTable>(m, "CpuSparseTable")
      .def(py::init<py::dict, int, bool, int, int>())
      .def("set_opt", &CpuSparseTable::set_opt)
      .def("pull", &CpuSparseTable::pull)
      .def("push", &CpuSparseTable::push)
      .def("size", &CpuSparseTable::size)
      .def("show_decay", &CpuSparseTable::show_decay)
      .def("dump", &CpuSparseTable::dump)
      .def("load_rows", &CpuSparseTable::load_rows)
      .def("clear", &CpuSparseTable::clear);
  py::class_<SparseDirWriter>(m, "SparseDirWriter")
      .def(py::init<const std::string&, const std::string&, int, int, bool, bool, float, int, int>())
      .def("append", &SparseDirWriter::append)
      .def("append_grouped", &SparseDirWriter::append_grouped)
      .def("close", &SparseDirWriter::close);
  py::class_<SparseBlockReader>(m, "SparseBlockReader")
      .def(py::init<const std::string&, int, int, bool>(), py::arg("path"), py::arg("kind"), py::arg("dim"), py::arg("use_cvm"))
      .def("next", &SparseBlockReader::next, py::arg("max_rows"))
      .def_property_readonly("is_binary", &SparseBlockReader::is_binary);
  py::class_<DictionaryReader>(m, "DictionaryReader")
      .def(py::init<const std::string&>())
      .def("next", &DictionaryReader::next, py::arg("max_rows"));
  m.def("dense_step", &dense_step);
  m.def("list_block_files", &list_block_files);
  m.def("unique_first_occurrence", &unique_first_occurrence);
  m.def("write_sparse_dir", &write_sparse_dir);
  m.def("read_sparse_dir", &read_sparse_dir);
  m.def("write_dense_file", &write_dense_file);
  m.def("read_dense_file", &read_dense_file);
  m.def("write_bn_file", &write_bn_file);
  m.def("read_bn_file", &read_bn_file);
  m.def("init_weights", &init_weights);
  m.def("owner_of", [](uint64_t s, int w) { return tn::owner_of(s, w); });
  m.def("block_of", [](uint64_t s) { return tn::block_of(s); });
  m.def("row_floats", [](int kind, int dim) { return tn::row_floats(kind, dim); });
}
