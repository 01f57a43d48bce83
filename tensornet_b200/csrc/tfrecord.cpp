// Native input pipeline for TFRecord files of tf.train.Example records (part of module _tn_cpu).
//
// The reference feeds its models through TensorFlow's C++ input pipeline: files sharded by rank, interleaved
// TFRecord readers, batches of serialized Examples parsed into sparse tensors (examples/common/util.py:23-39,
// examples/gen_example_data.py:20-60 for the record contents).  Here the same files are read without TensorFlow:
// worker threads own disjoint subsets of the files, interleave a few open readers each, parse the protobuf wire
// format by hand and hand over finished batches already in the slot-major layout the pull kernel takes
// (all ids of slot 0, then slot 1, ...; one offsets array over slots x examples), so a batch costs one
// host-to-device copy per array and no per-example Python work.
//
// File format (TensorFlow's record writer): per record  u64 length | u32 masked crc32c(length) | data |
// u32 masked crc32c(data), little endian; optionally the whole file gzip-compressed (zlib reads both kinds).
// Record contents: message Example { Features features = 1; }  Features { map<string, Feature> feature = 1; }
// Feature { oneof { BytesList bytes_list = 1; FloatList float_list = 2; Int64List int64_list = 3; } }, each list
// with `repeated value = 1` (packed or one element per tag).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <zlib.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace tfrec {

// ---------------------------------------------------------------------------------------------- crc32c
static uint32_t g_crc_table[8][256];
static std::once_flag g_crc_once;

static void crc_init() {
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
    g_crc_table[0][i] = c;
  }
  for (uint32_t i = 0; i < 256; ++i)
    for (int t = 1; t < 8; ++t) g_crc_table[t][i] = (g_crc_table[t - 1][i] >> 8) ^ g_crc_table[0][g_crc_table[t - 1][i] & 0xFF];
}

static uint32_t crc32c_sw(uint32_t crc, const uint8_t* p, size_t n) {
  std::call_once(g_crc_once, crc_init);
  while (n >= 8) {
    uint64_t v;
    std::memcpy(&v, p, 8);
    v ^= crc;
    crc = g_crc_table[7][v & 0xFF] ^ g_crc_table[6][(v >> 8) & 0xFF] ^ g_crc_table[5][(v >> 16) & 0xFF] ^
          g_crc_table[4][(v >> 24) & 0xFF] ^ g_crc_table[3][(v >> 32) & 0xFF] ^ g_crc_table[2][(v >> 40) & 0xFF] ^
          g_crc_table[1][(v >> 48) & 0xFF] ^ g_crc_table[0][(v >> 56) & 0xFF];
    p += 8;
    n -= 8;
  }
  while (n--) crc = (crc >> 8) ^ g_crc_table[0][(crc ^ *p++) & 0xFF];
  return crc;
}

#if defined(__x86_64__)
__attribute__((target("sse4.2"))) static uint32_t crc32c_hw(uint32_t crc, const uint8_t* p, size_t n) {
  uint64_t c = crc;
  while (n >= 8) {
    uint64_t v;
    std::memcpy(&v, p, 8);
    c = __builtin_ia32_crc32di(c, v);
    p += 8;
    n -= 8;
  }
  uint32_t c32 = (uint32_t)c;
  while (n--) c32 = __builtin_ia32_crc32qi(c32, *p++);
  return c32;
}
static bool have_hw_crc() {
  static const bool ok = __builtin_cpu_supports("sse4.2");
  return ok;
}
#endif

static uint32_t crc32c(const uint8_t* p, size_t n, bool allow_hw = true) {
  uint32_t c = 0xFFFFFFFFu;
#if defined(__x86_64__)
  if (allow_hw && have_hw_crc()) return ~crc32c_hw(c, p, n);
#endif
  (void)allow_hw;
  return ~crc32c_sw(c, p, n);
}

static inline uint32_t masked(uint32_t crc) { return ((crc >> 15) | (crc << 17)) + 0xa282ead8u; }

// ---------------------------------------------------------------------------------------------- record files
class RecordFile {
 public:
  // `path` is opened; `name` is what error messages call the file (the remote name of a fetched copy).
  explicit RecordFile(const std::string& path, const std::string& name) : path_(name), buf_(kChunk) {
    f_ = gzopen(path.c_str(), "rb");
    if (!f_) throw std::runtime_error("cannot open " + name);
    gzbuffer(f_, 1 << 18);
  }
  ~RecordFile() { if (f_) gzclose(f_); }
  RecordFile(const RecordFile&) = delete;
  RecordFile& operator=(const RecordFile&) = delete;

  // The next record, in place: `data` points into this reader's chunk buffer and stays valid until the next call.
  // False at a clean end of file.  A file that ends inside a record, or a checksum that does not match, raises.
  bool next(const uint8_t*& data, size_t& len_out, bool verify) {
    if (!want(12)) {
      if (end_ == pos_) return false;
      fail("ends inside a record header");
    }
    const uint8_t* head = buf_.data() + pos_;
    uint64_t len;
    uint32_t crc;
    std::memcpy(&len, head, 8);
    std::memcpy(&crc, head + 8, 4);
    if (masked(crc32c(head, 8)) != crc) fail("has a corrupt record length");
    if (len > (1ull << 31)) fail("has a record longer than 2 GiB");
    if (!want(12 + len + 4)) fail("ends inside a record");
    const uint8_t* rec = buf_.data() + pos_ + 12;
    if (verify) {
      uint32_t dcrc;
      std::memcpy(&dcrc, rec + len, 4);
      if (masked(crc32c(rec, len)) != dcrc) fail("has a record whose checksum does not match");
    }
    pos_ += 12 + len + 4;
    data = rec;
    len_out = len;
    return true;
  }

 private:
  static constexpr size_t kChunk = 1 << 20;

  // Makes `n` bytes available at pos_ (moving the unread tail to the front and reading on); false at end of file.
  bool want(size_t n) {
    if (end_ - pos_ >= n) return true;
    if (eof_) return false;
    if (pos_) {
      std::memmove(buf_.data(), buf_.data() + pos_, end_ - pos_);
      end_ -= pos_;
      pos_ = 0;
    }
    if (buf_.size() < n) buf_.resize(std::max(n, buf_.size() * 2));
    while (end_ < n || end_ < buf_.size()) {
      const size_t room = std::min<size_t>(buf_.size() - end_, 1u << 30);
      if (!room) break;
      const int r = gzread(f_, buf_.data() + end_, (unsigned)room);
      if (r < 0) fail("cannot be read (zlib error)");
      if (r == 0) { eof_ = true; break; }
      end_ += (size_t)r;
    }
    return end_ - pos_ >= n;
  }
  [[noreturn]] void fail(const char* what) { throw std::runtime_error("TFRecord file " + path_ + " " + what); }
  std::string path_;
  gzFile f_ = nullptr;
  std::vector<uint8_t> buf_;
  size_t pos_ = 0, end_ = 0;
  bool eof_ = false;
};

// ---------------------------------------------------------------------------------------------- protobuf wire format
struct Cursor {
  const uint8_t* p;
  const uint8_t* e;
  bool done() const { return p >= e; }
};

static inline bool varint(Cursor& c, uint64_t& v) {
  if (c.p < c.e && !(*c.p & 0x80)) {      // tags and short lengths: one byte
    v = *c.p++;
    return true;
  }
  if (c.e - c.p >= 10) {                  // ids: up to ten bytes, no bounds check per byte
    const uint8_t* p = c.p;
    uint64_t r = 0;
#pragma GCC unroll 10
    for (int i = 0; i < 10; ++i) {
      const uint64_t b = p[i];
      r |= (b & 0x7F) << (7 * i);
      if (!(b & 0x80)) {
        c.p = p + i + 1;
        v = r;
        return true;
      }
    }
    return false;
  }
  v = 0;
  for (int shift = 0; shift < 64 && c.p < c.e; shift += 7) {
    const uint8_t b = *c.p++;
    v |= (uint64_t)(b & 0x7F) << shift;
    if (!(b & 0x80)) return true;
  }
  return false;
}

static inline bool sub(Cursor& c, Cursor& out) {
  uint64_t n;
  if (!varint(c, n) || n > (uint64_t)(c.e - c.p)) return false;
  out.p = c.p;
  out.e = c.p + n;
  c.p += n;
  return true;
}

static inline bool skip(Cursor& c, uint32_t wire) {
  uint64_t v;
  Cursor s;
  switch (wire) {
    case 0: return varint(c, v);
    case 1: if (c.e - c.p < 8) return false; c.p += 8; return true;
    case 2: return sub(c, s);
    case 5: if (c.e - c.p < 4) return false; c.p += 4; return true;
    default: return false;
  }
}

// ---------------------------------------------------------------------------------------------- what to extract
struct Spec {
  std::vector<std::string> sparse;      // int64 features, any number of ids per example
  std::vector<std::string> dense;       // float features of a fixed width (int64 lists are converted)
  std::vector<int> dense_width, dense_off;
  std::vector<std::string> bytes;       // first bytes value per example
  std::string label;                    // first value of an int64 or float list; "" = none
  int dense_total = 0;
  bool single_hot = false;              // exactly one id per example and slot: missing -> default_id, extra ids dropped
  int64_t default_id = 0;
  std::unordered_map<std::string_view, int> index;

  void finish() {
    int code = 0;
    for (auto& s : sparse) index.emplace(std::string_view(s), code++);
    for (size_t j = 0; j < dense.size(); ++j) {
      dense_off.push_back(dense_total);
      dense_total += dense_width[j];
      index.emplace(std::string_view(dense[j]), code++);
    }
    if (!label.empty()) index.emplace(std::string_view(label), code);
    ++code;
    for (auto& s : bytes) index.emplace(std::string_view(s), code++);
    if ((size_t)index.size() != sparse.size() + dense.size() + bytes.size() + (label.empty() ? 0 : 1))
      throw std::invalid_argument("a feature name is listed twice");
  }
};

struct Batch {
  int n = 0;
  size_t S;
  size_t cap;                               // examples a full batch holds
  // While records arrive: ids in arrival order and, per (example, slot), where its ids start and how many there are
  // (with one id per slot the ids go straight to their place in `values` [S, cap] instead).
  std::vector<int64_t> ids;
  std::vector<uint32_t> pos;
  std::vector<int32_t> len;
  std::vector<float> dense, label;
  std::vector<std::vector<std::string>> bytes;
  // filled by seal(): the arrays handed to Python
  std::vector<int64_t> values;              // slot-major concatenation (or ids [S, n] when single_hot)
  std::vector<int32_t> offsets;             // [S * n + 1] over the concatenation
  std::vector<int32_t> local_offsets;       // [S, n + 1], every slot counted from 0
  std::vector<int64_t> slot_base;           // [S + 1] where each slot starts in `values`

  Batch(const Spec& sp, int expect, bool own_buffers = true) : S(sp.sparse.size()), cap((size_t)expect), bytes(sp.bytes.size()) {
    if (sp.single_hot) {
      values.assign(S * cap, sp.default_id);
    } else if (own_buffers) {                // otherwise hand_down() of the previous batch provides them
      ids.reserve((size_t)expect * S);
      pos.reserve((size_t)expect * S);
      len.reserve((size_t)expect * S);
    }
    dense.reserve((size_t)expect * sp.dense_total);
    label.reserve(sp.label.empty() ? 0 : (size_t)expect);
  }

  void seal(const Spec& sp) {
    slot_base.assign(S + 1, 0);
    if (ids.size() > (size_t)INT32_MAX) throw std::runtime_error("a batch holds more than 2^31 ids");
    if (sp.single_hot) {
      if ((size_t)n < cap)                     // a short last batch: close the gaps between the slots' rows
        for (size_t s = 1; s < S; ++s) std::memmove(values.data() + s * (size_t)n, values.data() + s * cap, (size_t)n * sizeof(int64_t));
      values.resize(S * (size_t)n);
      for (size_t s = 0; s < S; ++s) slot_base[s + 1] = (int64_t)((s + 1) * (size_t)n);
    } else {
      size_t total = 0;
      for (int32_t l : len) total += (size_t)l;
      values.resize(total);
      offsets.resize(S * (size_t)n + 1);
      local_offsets.resize(S * (size_t)(n + 1));
      size_t run = 0;
      for (size_t s = 0; s < S; ++s) {
        const size_t begin = run;
        for (int b = 0; b < n; ++b) {
          const size_t at = (size_t)b * S + s;
          offsets[s * n + b] = (int32_t)run;
          local_offsets[s * (n + 1) + b] = (int32_t)(run - begin);
          const int32_t l = len[at];
          const int64_t* src = ids.data() + pos[at];
          for (int32_t k = 0; k < l; ++k) values[run + k] = src[k];
          run += (size_t)l;
        }
        local_offsets[s * (n + 1) + n] = (int32_t)(run - begin);
        slot_base[s + 1] = (int64_t)run;
      }
      offsets[S * (size_t)n] = (int32_t)run;
    }
  }

  // The accumulation buffers of a sealed batch go on to the next one (their pages are already mapped).
  void hand_down(Batch& next) {
    ids.clear();
    pos.clear();
    len.clear();
    next.ids.swap(ids);
    next.pos.swap(pos);
    next.len.swap(len);
  }
};

// What a worker remembers between records: writers emit the features of every record in the same order, so the
// name at position i of the previous record predicts the name at position i of this one and most look-ups are one
// short comparison instead of a hash.
struct ParseState {
  std::vector<std::pair<std::string, int>> order;
};

// ---------------------------------------------------------------------------------------------- one Example
// The lists of a Feature.  `fn(kind, cursor)` sees the value list's bytes: kind 1 bytes, 2 float, 3 int64.
template <class F>
static bool for_each_list(Cursor feat, F&& fn) {
  while (!feat.done()) {
    uint64_t tag;
    if (!varint(feat, tag)) return false;
    const uint32_t field = (uint32_t)(tag >> 3), wire = (uint32_t)(tag & 7);
    if (wire == 2 && field >= 1 && field <= 3) {
      Cursor list;
      if (!sub(feat, list)) return false;
      if (!fn((int)field, list)) return false;
    } else if (!skip(feat, wire)) {
      return false;
    }
  }
  return true;
}

template <class F>
static bool for_each_int64(Cursor list, F&& fn) {
  while (!list.done()) {
    uint64_t tag, v;
    if (!varint(list, tag)) return false;
    const uint32_t field = (uint32_t)(tag >> 3), wire = (uint32_t)(tag & 7);
    if (field == 1 && wire == 2) {              // packed
      Cursor pk;
      if (!sub(list, pk)) return false;
      while (!pk.done()) {
        if (!varint(pk, v)) return false;
        fn((int64_t)v);
      }
    } else if (field == 1 && wire == 0) {       // one element per tag
      if (!varint(list, v)) return false;
      fn((int64_t)v);
    } else if (!skip(list, wire)) {
      return false;
    }
  }
  return true;
}

template <class F>
static bool for_each_float(Cursor list, F&& fn) {
  while (!list.done()) {
    uint64_t tag;
    if (!varint(list, tag)) return false;
    const uint32_t field = (uint32_t)(tag >> 3), wire = (uint32_t)(tag & 7);
    if (field == 1 && wire == 2) {
      Cursor pk;
      if (!sub(list, pk)) return false;
      if ((pk.e - pk.p) % 4) return false;
      for (; pk.p < pk.e; pk.p += 4) { float f; std::memcpy(&f, pk.p, 4); fn(f); }
    } else if (field == 1 && wire == 5) {
      if (list.e - list.p < 4) return false;
      float f;
      std::memcpy(&f, list.p, 4);
      list.p += 4;
      fn(f);
    } else if (!skip(list, wire)) {
      return false;
    }
  }
  return true;
}

static bool first_bytes(Cursor list, std::string& out) {
  while (!list.done()) {
    uint64_t tag;
    if (!varint(list, tag)) return false;
    const uint32_t field = (uint32_t)(tag >> 3), wire = (uint32_t)(tag & 7);
    if (field == 1 && wire == 2) {
      Cursor b;
      if (!sub(list, b)) return false;
      out.assign(reinterpret_cast<const char*>(b.p), (size_t)(b.e - b.p));
      return true;
    }
    if (!skip(list, wire)) return false;
  }
  return true;
}

// Fast path for a map entry of the usual shape: every length fits one byte, the name is the one the previous record
// had at this position, and the feature holds one list whose values sit in a single `value = 1` field (packed
// numbers, or one bytes value), or no values at all.  `p` points at the entry's length byte.  On success `kind` is
// the list (1 bytes, 2 float, 3 int64; 0 = feature without a list), [pay, pay + paylen) its value bytes and `total`
// the size of the entry including its length byte.  Anything else is left to the general parser.
static inline bool quick_entry(const uint8_t* p, const uint8_t* end, const std::string& key, int& kind,
                               const uint8_t*& pay, size_t& paylen, size_t& total) {
  const size_t kl = key.size();
  if (end - p < 1 || (p[0] & 0x80) || kl > 100) return false;
  const size_t L = p[0];
  if ((size_t)(end - p) < 1 + L || L < kl + 4) return false;
  const uint8_t* q = p + 1;
  if (q[0] != 0x0A || q[1] != kl || std::memcmp(q + 2, key.data(), kl) != 0) return false;
  const uint8_t* f = q + 2 + kl;
  const size_t F = L - kl - 4;                         // bytes of the Feature message
  if (f[0] != 0x12 || f[1] != F) return false;
  total = 1 + L;
  if (F == 0) { kind = 0; pay = f + 2; paylen = 0; return true; }
  if (F < 2 || f[3] != F - 2) return false;
  kind = f[2] == 0x0A ? 1 : f[2] == 0x12 ? 2 : f[2] == 0x1A ? 3 : 0;
  if (!kind) return false;
  if (F == 2) { pay = f + 4; paylen = 0; return true; }  // a list without values
  if (F < 4 || f[4] != 0x0A || f[5] != F - 4) return false;
  pay = f + 6;
  paylen = F - 4;
  return true;
}

// Varints filling [p, e) exactly; false when one runs past the end.
template <class F>
static inline bool packed_varints(const uint8_t* p, const uint8_t* e, F&& fn) {
  while (p < e) {
    uint64_t v = 0;
    int shift = 0;
    for (;;) {
      if (p >= e || shift > 63) return false;
      const uint64_t b = *p++;
      v |= (b & 0x7F) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
    }
    fn((int64_t)v);
  }
  return true;
}

// Stores the values of an entry that quick_entry() recognised; false (nothing stored) when they are not of a form
// this path handles, so that the general parser takes the entry.
static inline bool take_quick(const Spec& sp, Batch& b, int found, int kind, const uint8_t* pay, size_t paylen, size_t row,
                              size_t drow) {
  if (found < 0) return true;                            // a feature nobody asked for
  const size_t S = sp.sparse.size(), D = sp.dense.size(), code = (size_t)found;
  if (code < S && sp.single_hot) {                       // the first id, or the default when the list is empty
    int64_t first = sp.default_id;
    bool have = false;
    if (kind == 3 && !packed_varints(pay, pay + paylen, [&](int64_t x) { if (!have) { first = x; have = true; } })) return false;
    b.values[code * b.cap + (size_t)b.n] = first;
    return true;
  }
  if (code < S) {
    const size_t at = b.ids.size();
    if (kind == 3 && !packed_varints(pay, pay + paylen, [&](int64_t x) { b.ids.push_back(x); })) {
      b.ids.resize(at);
      return false;
    }
    b.pos[row + code] = (uint32_t)at;
    b.len[row + code] = (int32_t)(b.ids.size() - at);
    return true;
  }
  if (code < S + D) {
    const size_t j = code - S;
    float* out = b.dense.data() + drow + sp.dense_off[j];
    const int w = sp.dense_width[j];
    float tmp[64];
    if (w > 64) return false;
    int k = 0;
    if (kind == 2) {
      if (paylen % 4) return false;
      k = (int)std::min<size_t>((size_t)w, paylen / 4);
      std::memcpy(tmp, pay, (size_t)k * 4);
    } else if (kind == 3) {
      if (!packed_varints(pay, pay + paylen, [&](int64_t x) { if (k < w) tmp[k++] = (float)x; })) return false;
    }
    std::fill(out, out + w, 0.f);
    std::copy(tmp, tmp + k, out);
    return true;
  }
  if (code == S + D) {
    float y = 0.f;
    bool have = false;
    if (kind == 2) {
      if (paylen % 4) return false;
      if (paylen) { std::memcpy(&y, pay, 4); have = true; }
    } else if (kind == 3) {
      if (!packed_varints(pay, pay + paylen, [&](int64_t x) { if (!have) { y = (float)x; have = true; } })) return false;
    }
    if (have) b.label.back() = y;
    return true;
  }
  std::string& dst = b.bytes[code - S - D - 1].back();
  if (kind == 1 && paylen) dst.assign(reinterpret_cast<const char*>(pay), paylen);
  else if (kind == 1) return false;                      // an empty value or none: the general parser knows which
  return true;
}

// Adds one serialized Example to the batch.  Features that the record does not carry keep their defaults (no ids,
// zeros, label 0, empty bytes); when a name occurs twice the later entry wins, as in a protobuf map.
static void parse_example(const uint8_t* data, size_t len, const Spec& sp, Batch& b, ParseState& st) {
  const size_t S = sp.sparse.size(), D = sp.dense.size();
  const size_t row = b.pos.size();
  if (!sp.single_hot) {
    b.pos.resize(row + S, 0u);
    b.len.resize(row + S, 0);
  }
  const size_t drow = b.dense.size();
  b.dense.resize(drow + sp.dense_total, 0.f);
  if (!sp.label.empty()) b.label.push_back(0.f);
  for (auto& col : b.bytes) col.emplace_back();

  auto bad = []() { throw std::runtime_error("a record is not a well-formed tf.train.Example"); };
  size_t nth = 0;
  Cursor ex{data, data + len};
  while (!ex.done()) {
    uint64_t tag;
    if (!varint(ex, tag)) bad();
    if ((tag >> 3) != 1 || (tag & 7) != 2) { if (!skip(ex, (uint32_t)(tag & 7))) bad(); continue; }
    Cursor feats;
    if (!sub(ex, feats)) bad();
    while (!feats.done()) {
      if (!varint(feats, tag)) bad();
      if ((tag >> 3) != 1 || (tag & 7) != 2) { if (!skip(feats, (uint32_t)(tag & 7))) bad(); continue; }
      if (nth < st.order.size()) {
        int kind;
        const uint8_t* pay;
        size_t paylen, total;
        if (quick_entry(feats.p, feats.e, st.order[nth].first, kind, pay, paylen, total) &&
            take_quick(sp, b, st.order[nth].second, kind, pay, paylen, row, drow)) {
          feats.p += total;
          ++nth;
          continue;
        }
      }
      Cursor entry;
      if (!sub(feats, entry)) bad();
      std::string_view key;
      Cursor feat{nullptr, nullptr};
      while (!entry.done()) {
        if (!varint(entry, tag)) bad();
        Cursor f;
        if ((tag & 7) == 2 && ((tag >> 3) == 1 || (tag >> 3) == 2)) {
          if (!sub(entry, f)) bad();
          if ((tag >> 3) == 1) key = std::string_view(reinterpret_cast<const char*>(f.p), (size_t)(f.e - f.p));
          else feat = f;
        } else if (!skip(entry, (uint32_t)(tag & 7))) {
          bad();
        }
      }
      int found;
      if (nth < st.order.size() && st.order[nth].first.size() == key.size() &&
          std::memcmp(st.order[nth].first.data(), key.data(), key.size()) == 0) {
        found = st.order[nth].second;
      } else {
        const auto it = sp.index.find(key);
        found = it == sp.index.end() ? -1 : it->second;
        if (nth < 4096) {                       // remember the order of ordinary records only
          if (st.order.size() <= nth) st.order.resize(nth + 1);
          st.order[nth].first.assign(key.data(), key.size());
          st.order[nth].second = found;
        }
      }
      ++nth;
      if (found < 0) continue;
      const size_t code = (size_t)found;
      bool ok = true;
      if (code < S && sp.single_hot) {
        int64_t first = sp.default_id;
        bool have = false;
        ok = for_each_list(feat, [&](int kind, Cursor list) {
          if (kind != 3) return true;
          return for_each_int64(list, [&](int64_t x) { if (!have) { first = x; have = true; } });
        });
        b.values[code * b.cap + (size_t)b.n] = first;
      } else if (code < S) {
        const size_t at = b.ids.size();
        ok = for_each_list(feat, [&](int kind, Cursor list) {
          if (kind != 3) return true;
          return for_each_int64(list, [&](int64_t x) { b.ids.push_back(x); });
        });
        b.pos[row + code] = (uint32_t)at;
        b.len[row + code] = (int32_t)(b.ids.size() - at);
      } else if (code < S + D) {
        const size_t j = code - S;
        float* out = b.dense.data() + drow + sp.dense_off[j];
        const int w = sp.dense_width[j];
        int k = 0;
        std::fill(out, out + w, 0.f);
        ok = for_each_list(feat, [&](int kind, Cursor list) {
          if (kind == 2) return for_each_float(list, [&](float x) { if (k < w) out[k++] = x; });
          if (kind == 3) return for_each_int64(list, [&](int64_t x) { if (k < w) out[k++] = (float)x; });
          return true;
        });
      } else if (code == S + D) {
        bool have = false;
        float& y = b.label.back();
        ok = for_each_list(feat, [&](int kind, Cursor list) {
          if (kind == 2) return for_each_float(list, [&](float x) { if (!have) { y = x; have = true; } });
          if (kind == 3) return for_each_int64(list, [&](int64_t x) { if (!have) { y = (float)x; have = true; } });
          return true;
        });
      } else {
        std::string& dst = b.bytes[code - S - D - 1].back();
        ok = for_each_list(feat, [&](int kind, Cursor list) { return kind != 1 || first_bytes(list, dst); });
      }
      if (!ok) bad();
    }
  }
  ++b.n;
}

// ---------------------------------------------------------------------------------------------- workers
// A worker owns files w, w + W, w + 2W, ... of the list.  It keeps up to `cycle` of them open and takes `block`
// records from each in turn (the interleave of the reference's pipeline), cuts the record stream into batches and
// queues them.  Batches never mix records of two workers, so the order of the batches a reader hands out depends
// only on the file list and these parameters, not on thread timing.
struct Worker {
  std::vector<std::string> files;
  std::thread th;
  std::mutex mu;
  std::condition_variable can_put, can_get;
  std::deque<std::unique_ptr<Batch>> q;
  bool finished = false;
  std::string error;
};

class Batcher {
 public:
  Batcher(std::vector<std::string> files, int batch_size, std::vector<std::string> sparse, std::vector<std::string> dense,
          std::vector<int> dense_width, std::string label, std::vector<std::string> bytes, bool single_hot,
          int64_t default_id, bool drop_remainder, bool verify, int workers, int cycle, int block, int depth,
          py::object localize, py::object release)
      : batch_size_(batch_size), drop_remainder_(drop_remainder), verify_(verify), cycle_(std::max(1, cycle)),
        block_(std::max(1, block)), depth_(std::max(1, depth)), localize_(std::move(localize)), release_(std::move(release)) {
    hooks_ = !localize_.is_none();
    if (batch_size <= 0) throw std::invalid_argument("batch_size must be positive");
    if (dense.size() != dense_width.size()) throw std::invalid_argument("one width per dense feature");
    for (int w : dense_width) if (w <= 0) throw std::invalid_argument("dense widths must be positive");
    spec_.sparse = std::move(sparse);
    spec_.dense = std::move(dense);
    spec_.dense_width = std::move(dense_width);
    spec_.label = std::move(label);
    spec_.bytes = std::move(bytes);
    spec_.single_hot = single_hot;
    spec_.default_id = default_id;
    spec_.finish();
    const int W = std::max(1, std::min<int>(workers, (int)std::max<size_t>(1, files.size())));
    for (int w = 0; w < W; ++w) workers_.emplace_back(new Worker());
    for (size_t i = 0; i < files.size(); ++i) workers_[i % W]->files.push_back(files[i]);
    for (auto& w : workers_) {
      Worker* wp = w.get();
      wp->th = std::thread([this, wp] { run(wp); });
    }
  }

  ~Batcher() {
    // Workers may be waiting for the interpreter lock to call a hook: let go of it while they wind down.
    if (hooks_ && PyGILState_Check()) {
      py::gil_scoped_release nogil;
      close();
    } else {
      close();
    }
  }

  void close() {
    stop_.store(true);
    for (auto& w : workers_) {
      { std::lock_guard<std::mutex> g(w->mu); }
      w->can_put.notify_all();
      w->can_get.notify_all();
    }
    for (auto& w : workers_) if (w->th.joinable()) w->th.join();
  }

  // The next batch, or nullptr when every worker is done.  Workers are asked in turn; one that has finished is skipped.
  std::unique_ptr<Batch> next() {
    size_t idle = 0;
    while (idle < workers_.size()) {
      Worker& w = *workers_[turn_];
      turn_ = (turn_ + 1) % workers_.size();
      std::unique_lock<std::mutex> lk(w.mu);
      w.can_get.wait(lk, [&] { return !w.q.empty() || w.finished || stop_.load(); });
      if (!w.q.empty()) {
        auto b = std::move(w.q.front());
        w.q.pop_front();
        lk.unlock();
        w.can_put.notify_one();
        return b;
      }
      if (!w.error.empty()) throw std::runtime_error(w.error);
      if (stop_.load()) return nullptr;
      ++idle;
    }
    return nullptr;
  }

  const Spec& spec() const { return spec_; }

 private:
  bool put(Worker* w, std::unique_ptr<Batch> b) {
    std::unique_lock<std::mutex> lk(w->mu);
    w->can_put.wait(lk, [&] { return (int)w->q.size() < depth_ || stop_.load(); });
    if (stop_.load()) return false;
    w->q.push_back(std::move(b));
    lk.unlock();
    w->can_get.notify_one();
    return true;
  }

  void run(Worker* w) {
    try {
      std::vector<std::unique_ptr<RecordFile>> open;
      size_t next_file = 0;
      auto open_next = [&]() {
        const std::string& name = w->files[next_file++];
        return std::unique_ptr<RecordFile>(new RecordFile(hooks_ ? hook(localize_, name) : name, name));
      };
      std::vector<std::string> names;      // of the open files, for the release hook
      while ((int)open.size() < cycle_ && next_file < w->files.size()) {
        names.push_back(w->files[next_file]);
        open.push_back(open_next());
      }
      const uint8_t* rec = nullptr;
      size_t rec_len = 0;
      auto batch = std::make_unique<Batch>(spec_, batch_size_);
      ParseState state;
      size_t cur = 0;
      int in_block = 0;
      while (!open.empty() && !stop_.load()) {
        if (cur >= open.size()) cur = 0;
        if (!open[cur]->next(rec, rec_len, verify_)) {          // this file is done: the next unopened one takes its place
          open[cur].reset();
          if (hooks_) hook(release_, names[cur]);
          if (next_file < w->files.size()) {
            names[cur] = w->files[next_file];
            open[cur] = open_next();
          } else {
            open.erase(open.begin() + (long)cur);
            names.erase(names.begin() + (long)cur);
          }
          in_block = 0;
          continue;
        }
        parse_example(rec, rec_len, spec_, *batch, state);
        if (batch->n == batch_size_) {
          auto fresh = std::make_unique<Batch>(spec_, batch_size_, false);
          batch->seal(spec_);
          batch->hand_down(*fresh);
          if (!put(w, std::move(batch))) return;
          batch = std::move(fresh);
        }
        if (++in_block == block_) { in_block = 0; ++cur; }
      }
      if (batch->n > 0 && !drop_remainder_ && !stop_.load()) {
        batch->seal(spec_);
        put(w, std::move(batch));
      }
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> g(w->mu);
      w->error = e.what();
    }
    {
      std::lock_guard<std::mutex> g(w->mu);
      w->finished = true;
    }
    w->can_get.notify_all();
  }

  // Calls a Python hook from a worker thread; what it raises travels on as this worker's error.
  static std::string hook(const py::object& fn, const std::string& name) {
    py::gil_scoped_acquire gil;
    try {
      if (fn.is_none()) return name;
      py::object r = fn(name);
      return r.is_none() ? name : py::cast<std::string>(r);
    } catch (py::error_already_set& e) {
      const std::string what = e.what();
      e.restore();
      PyErr_Clear();
      throw std::runtime_error(what);
    }
  }

  Spec spec_;
  int batch_size_;
  bool drop_remainder_, verify_;
  int cycle_, block_, depth_;
  py::object localize_, release_;
  bool hooks_ = false;
  std::vector<std::unique_ptr<Worker>> workers_;
  std::atomic<bool> stop_{false};
  size_t turn_ = 0;
};

// ---------------------------------------------------------------------------------------------- writing
static void put_varint(std::string& out, uint64_t v) {
  while (v >= 0x80) { out.push_back((char)(v | 0x80)); v >>= 7; }
  out.push_back((char)v);
}

static void put_len_field(std::string& out, int field, const std::string& body) {
  put_varint(out, (uint64_t)(field << 3 | 2));
  put_varint(out, body.size());
  out += body;
}

// Serialized tf.train.Example from three dicts: name -> int64 array, name -> float32 array, name -> bytes.
static py::bytes encode_example(const py::dict& ints, const py::dict& floats, const py::dict& raw) {
  std::string features;
  auto entry = [&](const std::string& key, int list_field, const std::string& list) {
    std::string feature, e;
    put_len_field(feature, list_field, list);
    put_len_field(e, 1, key);
    put_len_field(e, 2, feature);
    put_len_field(features, 1, e);
  };
  for (auto kv : ints) {
    auto arr = py::array_t<int64_t, py::array::c_style | py::array::forcecast>::ensure(kv.second);
    if (!arr) throw std::invalid_argument("int64 features must convert to an int64 array");
    std::string packed, list;
    for (py::ssize_t i = 0; i < arr.size(); ++i) put_varint(packed, (uint64_t)arr.data()[i]);
    if (arr.size()) put_len_field(list, 1, packed);
    entry(py::cast<std::string>(kv.first), 3, list);
  }
  for (auto kv : floats) {
    auto arr = py::array_t<float, py::array::c_style | py::array::forcecast>::ensure(kv.second);
    if (!arr) throw std::invalid_argument("float features must convert to a float32 array");
    std::string list;
    if (arr.size()) put_len_field(list, 1, std::string(reinterpret_cast<const char*>(arr.data()), (size_t)arr.size() * 4));
    entry(py::cast<std::string>(kv.first), 2, list);
  }
  for (auto kv : raw) {
    std::string list;
    put_len_field(list, 1, py::cast<std::string>(kv.second));
    entry(py::cast<std::string>(kv.first), 1, list);
  }
  std::string example;
  put_len_field(example, 1, features);
  return py::bytes(example);
}

class Writer {
 public:
  Writer(const std::string& path, bool gzip) : path_(path) {
    if (gzip) gz_ = gzopen(path.c_str(), "wb6"); else fp_ = std::fopen(path.c_str(), "wb");
    if (!gz_ && !fp_) throw std::runtime_error("cannot create " + path);
  }
  ~Writer() { try { close(); } catch (...) {} }
  void write(const std::string& rec) {
    uint8_t head[12];
    const uint64_t len = rec.size();
    std::memcpy(head, &len, 8);
    const uint32_t c1 = masked(crc32c(head, 8));
    std::memcpy(head + 8, &c1, 4);
    const uint32_t c2 = masked(crc32c(reinterpret_cast<const uint8_t*>(rec.data()), rec.size()));
    raw(head, 12);
    raw(rec.data(), rec.size());
    raw(&c2, 4);
  }
  void close() {
    int rc = 0;
    if (gz_) { rc = gzclose(gz_); gz_ = nullptr; }
    if (fp_) { rc = std::fclose(fp_); fp_ = nullptr; }
    if (rc != 0) throw std::runtime_error("closing " + path_ + " failed");
  }

 private:
  void raw(const void* p, size_t n) {
    if (!gz_ && !fp_) throw std::runtime_error(path_ + " is closed");
    const bool ok = gz_ ? (n == 0 || gzwrite(gz_, p, (unsigned)n) == (int)n) : std::fwrite(p, 1, n, fp_) == n;
    if (!ok) throw std::runtime_error("writing " + path_ + " failed");
  }
  std::string path_;
  gzFile gz_ = nullptr;
  FILE* fp_ = nullptr;
};

// ---------------------------------------------------------------------------------------------- Python side
template <class T>
static py::array_t<T> take(std::vector<T>&& v, std::vector<py::ssize_t> shape) {
  auto* h = new std::vector<T>(std::move(v));
  py::capsule owner(h, [](void* p) { delete static_cast<std::vector<T>*>(p); });
  std::vector<py::ssize_t> strides(shape.size());
  py::ssize_t st = (py::ssize_t)sizeof(T);
  for (size_t i = shape.size(); i-- > 0;) { strides[i] = st; st *= shape[i]; }
  return py::array_t<T>(shape, strides, h->data(), owner);
}

static py::object next_batch(Batcher& self) {
  std::unique_ptr<Batch> b;
  {
    py::gil_scoped_release nogil;
    b = self.next();
  }
  if (!b) return py::none();
  const Spec& sp = self.spec();
  const py::ssize_t n = b->n, S = (py::ssize_t)sp.sparse.size();
  py::dict out;
  out["n"] = n;
  if (sp.single_hot) {
    out["ids"] = take(std::move(b->values), {S, n});
  } else {
    out["values"] = take(std::move(b->values), {(py::ssize_t)b->values.size()});
    out["offsets"] = take(std::move(b->offsets), {S * n + 1});
    out["local_offsets"] = take(std::move(b->local_offsets), {S, n + 1});
  }
  out["slot_base"] = take(std::move(b->slot_base), {S + 1});
  if (sp.dense_total) out["dense"] = take(std::move(b->dense), {n, (py::ssize_t)sp.dense_total});
  if (!sp.label.empty()) out["label"] = take(std::move(b->label), {n});
  for (size_t k = 0; k < sp.bytes.size(); ++k) {
    py::list col;
    for (auto& s : b->bytes[k]) col.append(py::bytes(s));
    out[py::str(sp.bytes[k])] = col;
  }
  return out;
}

}  // namespace tfrec

void bind_tfrecord(py::module_& m) {
  using namespace tfrec;
  py::class_<Batcher>(m, "TFRecordBatcher")
      .def(py::init<std::vector<std::string>, int, std::vector<std::string>, std::vector<std::string>, std::vector<int>,
                    std::string, std::vector<std::string>, bool, int64_t, bool, bool, int, int, int, int, py::object, py::object>(),
           py::arg("files"), py::arg("batch_size"), py::arg("sparse"), py::arg("dense"), py::arg("dense_width"),
           py::arg("label"), py::arg("bytes"), py::arg("single_hot"), py::arg("default_id"), py::arg("drop_remainder"),
           py::arg("verify"), py::arg("workers"), py::arg("cycle"), py::arg("block"), py::arg("depth"),
           py::arg("localize") = py::none(), py::arg("release") = py::none())
      .def("next", &next_batch)
      .def("close", [](Batcher& b) { py::gil_scoped_release nogil; b.close(); });
  py::class_<Writer>(m, "TFRecordWriter")
      .def(py::init<const std::string&, bool>(), py::arg("path"), py::arg("gzip") = false)
      .def("write", [](Writer& w, const py::bytes& rec) { w.write(rec); })
      .def("close", &Writer::close);
  m.def("tf_example_encode", &encode_example, py::arg("ints"), py::arg("floats") = py::dict(), py::arg("raw") = py::dict());
  m.def("crc32c", [](const py::bytes& b, bool hw) {
    const std::string s = b;
    return crc32c(reinterpret_cast<const uint8_t*>(s.data()), s.size(), hw);
  }, py::arg("data"), py::arg("hw") = true);
  m.def("tf_masked_crc32c", [](const py::bytes& b) {
    const std::string s = b;
    return masked(crc32c(reinterpret_cast<const uint8_t*>(s.data()), s.size()));
  });
}
