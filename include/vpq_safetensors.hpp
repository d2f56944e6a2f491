// vpq_safetensors.hpp -- on-disk format of a quantized checkpoint: writer and reader for the
// (weight U32, scales F16, biases F16) triples the reference's model-quantize tool emits.
// Header-only, host-only (no CUDA).
//
//   reference (generative-models/quantize, llama3)              here (namespace vpq::host)
//   SafetensorsWriter::add / close   safetensors-writer.h:22-39   SafetensorsWriter::add / close
//   MetalLlamaWeights::open_model    metal-llama-weights.h:47-57  SafetensorsReader::open_model
//   quant_2d_buf output naming       model-quantizer.cc:1265-1272 write_quant_linear / read_quant_linear
//   config.json "quantization"       model-quantizer.cc:1991-1997 write_quant_config / read_quant_config
//
// Format. A model directory holds shards `model-%05d-of-%05d.safetensors`, an index
// `model.safetensors.index.json` {"metadata":{"total_size":0},"weight_map":{name: shard}} and a
// `config.json` with a top-level "quantization":{"group_size":G,"bits":B}. A shard is
// [u64 little-endian header length][JSON header][data blob]; header entries are
// "name":{"dtype":"U32|F16|BF16|F32|...","shape":[...],"data_offsets":[begin,end]} relative to the
// blob; the header is right-padded with spaces so that the blob starts 16-byte aligned; tensors
// tile the blob without gaps, and small tensors whose size is not a multiple of 16 go to the end
// of their shard so that everything before them stays 16-byte aligned.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

namespace vpq {
namespace host {

namespace st_detail {

inline std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') {
      o += '\\';
      o += c;
    } else if (static_cast<unsigned char>(c) < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "\\u%04x", c);
      o += buf;
    } else {
      o += c;
    }
  }
  return o;
}

inline std::string shard_name(int idx, int total) {
  char buf[64];
  std::snprintf(buf, sizeof(buf), "model-%05d-of-%05d.safetensors", idx, total);
  return buf;
}

// The few JSON forms these files use: objects, arrays, strings, integers. A cursor over text.
struct Cursor {
  const std::string& s;
  size_t i = 0;
  bool ok = true;
  explicit Cursor(const std::string& text) : s(text) {}
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) { ++i; }
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) {
      ++i;
      return true;
    }
    return false;
  }
  bool peek(char c) {
    ws();
    return i < s.size() && s[i] == c;
  }
  std::string str() {
    std::string o;
    ws();
    if (i >= s.size() || s[i] != '"') {
      ok = false;
      return o;
    }
    for (++i; i < s.size() && s[i] != '"'; ++i) {
      if (s[i] == '\\' && i + 1 < s.size()) {
        ++i;
        if (s[i] == 'u' && i + 4 < s.size()) {  // control characters only: keep the low byte
          o += static_cast<char>(std::strtol(s.substr(i + 1, 4).c_str(), nullptr, 16));
          i += 4;
          continue;
        }
        o += s[i] == 'n' ? '\n' : s[i] == 't' ? '\t' : s[i];
      } else {
        o += s[i];
      }
    }
    if (i >= s.size()) { ok = false; }
    ++i;
    return o;
  }
  int64_t integer() {
    ws();
    size_t j = i;
    if (j < s.size() && s[j] == '-') { ++j; }
    while (j < s.size() && s[j] >= '0' && s[j] <= '9') { ++j; }
    if (j == i) {
      ok = false;
      return 0;
    }
    const int64_t v = std::strtoll(s.substr(i, j - i).c_str(), nullptr, 10);
    i = j;
    return v;
  }
  // Skips any value (used for fields this reader does not need).
  void skip() {
    ws();
    if (i >= s.size()) {
      ok = false;
      return;
    }
    if (s[i] == '"') {
      str();
    } else if (s[i] == '{' || s[i] == '[') {
      const char close = s[i] == '{' ? '}' : ']';
      ++i;
      while (ok && !peek(close)) {
        if (close == '}') {
          str();
          if (!eat(':')) { ok = false; }
        }
        skip();
        if (!eat(',')) { break; }
      }
      if (!eat(close)) { ok = false; }
    } else {
      while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') { ++i; }
    }
  }
};

inline bool read_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) { return false; }
  std::ostringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  return true;
}

}  // namespace st_detail

// Appends tensors to shards of at most `shard_max_bytes` of data; the bytes are written to the
// shard's data file as they arrive (the pointer need not outlive add()). close() assembles
// header + data into the final shard files and writes the index.
class SafetensorsWriter {
 public:
  explicit SafetensorsWriter(std::string out_dir, uint64_t shard_max_bytes = 5ull << 30)
      : _dir(std::move(out_dir)), _max(shard_max_bytes) {}
  SafetensorsWriter(const SafetensorsWriter&) = delete;
  SafetensorsWriter& operator=(const SafetensorsWriter&) = delete;
  ~SafetensorsWriter() { close(); }

  bool add(const std::string& name, const std::string& dtype, const std::vector<int64_t>& shape,
           const void* data, uint64_t nbytes) {
    if (_closed || _failed || (!data && nbytes)) { return false; }
    if (_shards.empty() || (_shards.back().size + _shards.back().deferred_bytes > 0 &&
                            _shards.back().size + _shards.back().deferred_bytes + nbytes > _max)) {
      if (!open_shard()) { return false; }
    }
    Shard& sh = _shards.back();
    Entry e{name, dtype, shape, 0, nbytes};
    // a small tensor whose size would knock its successors off the 16-byte grid waits for the end
    if ((nbytes % 16) != 0 && nbytes <= kDeferMax && sh.deferred_bytes + nbytes <= kDeferTotalMax) {
      Deferred d;
      d.e = e;
      d.bytes.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + nbytes);
      sh.deferred_bytes += nbytes;
      sh.deferred.push_back(std::move(d));
      return true;
    }
    e.offset = sh.size;
    sh.data.write(static_cast<const char*>(data), static_cast<std::streamsize>(nbytes));
    if (!sh.data) {
      _failed = true;
      return false;
    }
    sh.size += nbytes;
    sh.entries.push_back(std::move(e));
    return true;
  }

  bool close() {
    if (_closed) { return !_failed; }
    _closed = true;
    const int total = static_cast<int>(_shards.size());
    std::string index = "{\"metadata\":{\"total_size\":0},\"weight_map\":{";
    bool first = true;
    for (int i = 0; i < total && !_failed; ++i) {
      Shard& sh = _shards[i];
      for (Deferred& d : sh.deferred) {
        d.e.offset = sh.size;
        sh.data.write(reinterpret_cast<const char*>(d.bytes.data()), static_cast<std::streamsize>(d.bytes.size()));
        sh.size += d.bytes.size();
        sh.entries.push_back(d.e);
      }
      sh.data.close();
      const std::string fname = st_detail::shard_name(i + 1, total);
      if (!finalize(sh, _dir + "/" + fname)) {
        _failed = true;
        break;
      }
      for (const Entry& e : sh.entries) {
        index += (first ? "\"" : ",\"") + st_detail::json_escape(e.name) + "\":\"" + fname + "\"";
        first = false;
      }
    }
    index += "}}";
    if (!_failed) {
      std::ofstream f(_dir + "/model.safetensors.index.json", std::ios::binary);
      f << index;
      if (!f) { _failed = true; }
    }
    return !_failed;
  }

 private:
  struct Entry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    uint64_t offset, nbytes;
  };
  struct Deferred {
    Entry e;
    std::vector<uint8_t> bytes;
  };
  struct Shard {
    std::string tmp_path;
    std::ofstream data;
    uint64_t size = 0;
    std::vector<Entry> entries;
    std::vector<Deferred> deferred;
    uint64_t deferred_bytes = 0;
  };
  static constexpr uint64_t kDeferMax = 1ull << 20;
  static constexpr uint64_t kDeferTotalMax = 64ull << 20;

  bool open_shard() {
    _shards.emplace_back();
    Shard& sh = _shards.back();
    sh.tmp_path = _dir + "/.shard-" + std::to_string(_shards.size()) + ".data.tmp";
    sh.data.open(sh.tmp_path, std::ios::binary | std::ios::trunc);
    if (!sh.data) {
      _failed = true;
      return false;
    }
    return true;
  }

  bool finalize(Shard& sh, const std::string& path) {
    std::string hdr = "{";
    for (size_t k = 0; k < sh.entries.size(); ++k) {
      const Entry& e = sh.entries[k];
      hdr += (k ? ",\"" : "\"") + st_detail::json_escape(e.name) + "\":{\"dtype\":\"" + e.dtype + "\",\"shape\":[";
      for (size_t d = 0; d < e.shape.size(); ++d) { hdr += (d ? "," : "") + std::to_string(e.shape[d]); }
      hdr += "],\"data_offsets\":[" + std::to_string(e.offset) + "," + std::to_string(e.offset + e.nbytes) + "]}";
    }
    hdr += "}";
    while ((8 + hdr.size()) % 16 != 0) { hdr += ' '; }  // the blob starts 16-byte aligned
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    const uint64_t n = hdr.size();
    unsigned char len[8];
    for (int b = 0; b < 8; ++b) { len[b] = static_cast<unsigned char>(n >> (8 * b)); }
    out.write(reinterpret_cast<const char*>(len), 8);
    out.write(hdr.data(), static_cast<std::streamsize>(hdr.size()));
    std::ifstream in(sh.tmp_path, std::ios::binary);
    std::vector<char> buf(1 << 20);
    while (in) {
      in.read(buf.data(), static_cast<std::streamsize>(buf.size()));
      out.write(buf.data(), in.gcount());
    }
    in.close();
    std::remove(sh.tmp_path.c_str());
    return static_cast<bool>(out);
  }

  std::string _dir;
  uint64_t _max;
  std::vector<Shard> _shards;
  bool _closed = false, _failed = false;
};

// One tensor of an opened model directory (or single shard file).
struct TensorInfo {
  std::string dtype;
  std::vector<int64_t> shape;
  std::string file;        // shard path
  uint64_t begin = 0;      // absolute byte range in the shard file
  uint64_t nbytes = 0;
  bool aligned16() const { return (begin % 16) == 0; }
};

class SafetensorsReader {
 public:
  // Opens every shard the index names (or, without an index, a single `model.safetensors`).
  bool open_model(const std::string& dir) {
    _tensors.clear();
    std::string idx;
    if (st_detail::read_file(dir + "/model.safetensors.index.json", &idx)) {
      st_detail::Cursor c(idx);
      std::map<std::string, bool> shards;
      if (!c.eat('{')) { return false; }
      while (c.ok && !c.peek('}')) {
        const std::string key = c.str();
        if (!c.eat(':')) { return false; }
        if (key == "weight_map") {
          if (!c.eat('{')) { return false; }
          while (c.ok && !c.peek('}')) {
            c.str();
            if (!c.eat(':')) { return false; }
            shards[c.str()] = true;
            if (!c.eat(',')) { break; }
          }
          if (!c.eat('}')) { return false; }
        } else {
          c.skip();
        }
        if (!c.eat(',')) { break; }
      }
      if (!c.ok) { return false; }
      for (const auto& kv : shards) {
        if (!open_shard(dir + "/" + kv.first)) { return false; }
      }
      return true;
    }
    return open_shard(dir + "/model.safetensors");
  }

  bool open_shard(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    unsigned char len[8];
    if (!f.read(reinterpret_cast<char*>(len), 8)) { return false; }
    uint64_t n = 0;
    for (int b = 0; b < 8; ++b) { n |= static_cast<uint64_t>(len[b]) << (8 * b); }
    if (n == 0 || n > (1ull << 31)) { return false; }
    std::string hdr(n, '\0');
    if (!f.read(&hdr[0], static_cast<std::streamsize>(n))) { return false; }
    f.seekg(0, std::ios::end);
    const uint64_t file_size = static_cast<uint64_t>(f.tellg());
    const uint64_t blob = 8 + n;
    st_detail::Cursor c(hdr);
    if (!c.eat('{')) { return false; }
    while (c.ok && !c.peek('}')) {
      const std::string name = c.str();
      if (!c.eat(':')) { return false; }
      if (name == "__metadata__") {
        c.skip();
      } else {
        TensorInfo t;
        t.file = path;
        uint64_t b0 = 0, b1 = 0;
        if (!c.eat('{')) { return false; }
        while (c.ok && !c.peek('}')) {
          const std::string k = c.str();
          if (!c.eat(':')) { return false; }
          if (k == "dtype") {
            t.dtype = c.str();
          } else if (k == "shape") {
            if (!c.eat('[')) { return false; }
            while (c.ok && !c.peek(']')) {
              t.shape.push_back(c.integer());
              if (!c.eat(',')) { break; }
            }
            if (!c.eat(']')) { return false; }
          } else if (k == "data_offsets") {
            if (!c.eat('[')) { return false; }
            b0 = static_cast<uint64_t>(c.integer());
            if (!c.eat(',')) { return false; }
            b1 = static_cast<uint64_t>(c.integer());
            if (!c.eat(']')) { return false; }
          } else {
            c.skip();
          }
          if (!c.eat(',')) { break; }
        }
        if (!c.eat('}')) { return false; }
        if (b1 < b0 || blob + b1 > file_size) { return false; }  // a range outside the file
        t.begin = blob + b0;
        t.nbytes = b1 - b0;
        _tensors[name] = std::move(t);
      }
      if (!c.eat(',')) { break; }
    }
    return c.ok;
  }

  const TensorInfo* find(const std::string& name) const {
    auto it = _tensors.find(name);
    return it == _tensors.end() ? nullptr : &it->second;
  }
  const std::map<std::string, TensorInfo>& tensors() const { return _tensors; }

  // Copies a tensor's bytes into dst (capacity >= nbytes).
  bool read(const TensorInfo& t, void* dst) const {
    std::ifstream f(t.file, std::ios::binary);
    f.seekg(static_cast<std::streamoff>(t.begin));
    return static_cast<bool>(f.read(static_cast<char*>(dst), static_cast<std::streamsize>(t.nbytes)));
  }

 private:
  std::map<std::string, TensorInfo> _tensors;
};

// One quantized linear on the host, as stored: codes U32 [N, K*bits/32], scales / biases F16 [N, K/group].
struct QuantLinear {
  int64_t N = 0, K = 0;
  int bits = 0, group = 0;
  std::vector<uint32_t> weight;
  std::vector<uint16_t> scales, biases;
};

// `<pfx>.weight`, `<pfx>.scales`, `<pfx>.biases` (generative-models/quantize/model-quantizer.cc:1265-1272).
inline bool write_quant_linear(SafetensorsWriter& w, const std::string& pfx, const QuantLinear& q) {
  const int64_t wc = q.K * q.bits / 32, gc = q.K / q.group;
  if (q.N <= 0 || q.K <= 0 || q.bits <= 0 || q.group <= 0 || (q.K % q.group) != 0 ||
      static_cast<int64_t>(q.weight.size()) != q.N * wc || static_cast<int64_t>(q.scales.size()) != q.N * gc ||
      q.biases.size() != q.scales.size()) {
    return false;
  }
  return w.add(pfx + ".weight", "U32", {q.N, wc}, q.weight.data(), q.weight.size() * 4) &&
         w.add(pfx + ".scales", "F16", {q.N, gc}, q.scales.data(), q.scales.size() * 2) &&
         w.add(pfx + ".biases", "F16", {q.N, gc}, q.biases.data(), q.biases.size() * 2);
}

// Reads the triple back. The group size comes from config.json (or the caller); K and the bit
// width follow from the shapes: K = scales_cols * group, bits = weight_cols * 32 / K
// (docs/PLUGINS.md:218-220, generative-models/flux2/metal-flux2-transformer.cc:131-136), which is
// how per-tensor mixed widths load.
inline bool read_quant_linear(const SafetensorsReader& r, const std::string& pfx, int group, QuantLinear* q) {
  const TensorInfo* tw = r.find(pfx + ".weight");
  const TensorInfo* ts = r.find(pfx + ".scales");
  const TensorInfo* tb = r.find(pfx + ".biases");
  if (!tw || !ts || !tb || group <= 0) { return false; }
  if (tw->dtype != "U32" || ts->dtype != "F16" || tb->dtype != "F16" || tw->shape.size() != 2 ||
      ts->shape.size() != 2 || tb->shape != ts->shape || tw->shape[0] != ts->shape[0]) {
    return false;
  }
  q->N = tw->shape[0];
  q->K = ts->shape[1] * group;
  q->group = group;
  if (q->K <= 0 || (tw->shape[1] * 32) % q->K != 0) { return false; }
  q->bits = static_cast<int>(tw->shape[1] * 32 / q->K);
  if (tw->nbytes != static_cast<uint64_t>(q->N * tw->shape[1] * 4) ||
      ts->nbytes != static_cast<uint64_t>(q->N * ts->shape[1] * 2) || tb->nbytes != ts->nbytes) {
    return false;
  }
  q->weight.resize(tw->nbytes / 4);
  q->scales.resize(ts->nbytes / 2);
  q->biases.resize(tb->nbytes / 2);
  return r.read(*tw, q->weight.data()) && r.read(*ts, q->scales.data()) && r.read(*tb, q->biases.data());
}

// config.json with the top-level "quantization" object (model-quantizer.cc:1991-1997). If the
// directory already holds a config.json, the key is added to it (or replaced).
inline bool write_quant_config(const std::string& dir, int group, int bits) {
  const std::string q = "\"quantization\":{\"group_size\":" + std::to_string(group) + ",\"bits\":" + std::to_string(bits) + "}";
  std::string text;
  if (st_detail::read_file(dir + "/config.json", &text)) {
    const size_t at = text.find("\"quantization\"");
    if (at != std::string::npos) {
      const size_t close = text.find('}', at);
      if (close == std::string::npos) { return false; }
      text.replace(at, close + 1 - at, q);
    } else {
      const size_t last = text.rfind('}');
      if (last == std::string::npos) { return false; }
      size_t prev = last;
      while (prev > 0 && (text[prev - 1] == ' ' || text[prev - 1] == '\n' || text[prev - 1] == '\t' || text[prev - 1] == '\r')) { --prev; }
      const bool empty_obj = prev > 0 && text[prev - 1] == '{';
      text.insert(last, (empty_obj ? "" : ",") + q);
    }
  } else {
    text = "{" + q + "}";
  }
  std::ofstream f(dir + "/config.json", std::ios::binary | std::ios::trunc);
  f << text;
  return static_cast<bool>(f);
}

inline bool read_quant_config(const std::string& dir, int* group, int* bits) {
  std::string text;
  if (!st_detail::read_file(dir + "/config.json", &text)) { return false; }
  st_detail::Cursor c(text);
  if (!c.eat('{')) { return false; }
  while (c.ok && !c.peek('}')) {
    const std::string key = c.str();
    if (!c.eat(':')) { return false; }
    if (key == "quantization") {
      if (!c.eat('{')) { return false; }
      int g = 0, b = 0;
      while (c.ok && !c.peek('}')) {
        const std::string k = c.str();
        if (!c.eat(':')) { return false; }
        if (k == "group_size") {
          g = static_cast<int>(c.integer());
        } else if (k == "bits") {
          b = static_cast<int>(c.integer());
        } else {
          c.skip();
        }
        if (!c.eat(',')) { break; }
      }
      if (!c.ok || g <= 0 || b <= 0) { return false; }
      *group = g;
      *bits = b;
      return true;
    }
    c.skip();
    if (!c.eat(',')) { break; }
  }
  return false;
}

}  // namespace host
}  // namespace vpq
