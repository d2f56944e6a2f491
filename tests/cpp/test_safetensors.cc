// CPU test of include/vpq_safetensors.hpp in the style of the reference's writer tests
// (tests/unit-tests/model-quantize-roundtrip.cc:84-164 byte-identical writer <-> reader,
// :182-231 aligned data section, :247-325 odd-sized tensors deferred, ranges tile the blob).
// usage: test_safetensors <scratch dir>   (the Python test then re-parses what was written)
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <sys/stat.h>
#include <vector>

#include "vpq_safetensors.hpp"

using namespace vpq::host;

static int g_failed = 0;
#define EXPECT(cond)                                                       \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
      ++g_failed;                                                          \
    }                                                                      \
  } while (0)

static uint32_t lcg(uint32_t& s) { return s = s * 1664525u + 1013904223u; }

static QuantLinear make_linear(int64_t N, int64_t K, int bits, int group, uint32_t seed) {
  QuantLinear q;
  q.N = N;
  q.K = K;
  q.bits = bits;
  q.group = group;
  q.weight.resize(N * (K * bits / 32));
  q.scales.resize(N * (K / group));
  q.biases.resize(N * (K / group));
  for (auto& v : q.weight) { v = lcg(seed); }
  for (auto& v : q.scales) { v = static_cast<uint16_t>(0x2000 + (lcg(seed) >> 20)); }
  for (auto& v : q.biases) { v = static_cast<uint16_t>(0xa000 + (lcg(seed) >> 20)); }
  return q;
}

static bool same(const QuantLinear& a, const QuantLinear& b) {
  return a.N == b.N && a.K == b.K && a.bits == b.bits && a.group == b.group && a.weight == b.weight &&
         a.scales == b.scales && a.biases == b.biases;
}

static void test_roundtrip_two_shards(const std::string& dir) {
  mkdir(dir.c_str(), 0755);
  const QuantLinear q4 = make_linear(48, 256, 4, 64, 11), q8 = make_linear(16, 128, 8, 64, 12),
                    big = make_linear(64, 512, 4, 64, 13);
  const uint16_t scalar = 0x3c00;
  const float norm[5] = {1.f, 2.f, 3.f, 4.f, 5.f};  // 20 bytes: not a multiple of 16
  {
    SafetensorsWriter wr(dir, /*shard_max_bytes=*/12000);
    EXPECT(write_quant_linear(wr, "model.layers.0.self_attn.q_proj", q4));
    EXPECT(wr.add("model.layers.0.layer_scalar", "F16", {1}, &scalar, 2));
    EXPECT(write_quant_linear(wr, "model.layers.0.mlp.down_proj", q8));
    EXPECT(wr.add("model.norm.weight", "F32", {5}, norm, sizeof(norm)));
    EXPECT(write_quant_linear(wr, "model.layers.1.mlp.up_proj", big));
    EXPECT(wr.close());
    EXPECT(!wr.add("late", "F16", {1}, &scalar, 2));  // unusable after close
  }
  EXPECT(write_quant_config(dir, 64, 4));
  int g = 0, b = 0;
  EXPECT(read_quant_config(dir, &g, &b) && g == 64 && b == 4);

  SafetensorsReader rd;
  EXPECT(rd.open_model(dir));
  EXPECT(rd.tensors().size() == 11);
  QuantLinear r4, r8, rbig;
  EXPECT(read_quant_linear(rd, "model.layers.0.self_attn.q_proj", g, &r4) && same(r4, q4));
  EXPECT(read_quant_linear(rd, "model.layers.0.mlp.down_proj", g, &r8) && same(r8, q8));  // bits inferred: 8
  EXPECT(read_quant_linear(rd, "model.layers.1.mlp.up_proj", g, &rbig) && same(rbig, big));
  EXPECT(r8.bits == 8 && r4.bits == 4);
  EXPECT(!read_quant_linear(rd, "model.layers.9.nothing", g, &r4));
  // every tensor whose size is a multiple of 16 starts on a 16-byte boundary of its file
  std::map<std::string, std::vector<std::pair<uint64_t, uint64_t>>> per_file;
  for (const auto& kv : rd.tensors()) {
    if (kv.second.nbytes % 16 == 0) { EXPECT(kv.second.aligned16()); }
    per_file[kv.second.file].push_back({kv.second.begin, kv.second.begin + kv.second.nbytes});
  }
  EXPECT(per_file.size() >= 2);  // the byte budget split the model
  for (auto& kv : per_file) {    // ranges tile each blob without gaps
    std::sort(kv.second.begin(), kv.second.end());
    for (size_t i = 1; i < kv.second.size(); ++i) { EXPECT(kv.second[i].first == kv.second[i - 1].second); }
  }
  float back[5] = {0};
  const TensorInfo* t = rd.find("model.norm.weight");
  EXPECT(t && t->dtype == "F32" && t->shape.size() == 1 && t->shape[0] == 5 && rd.read(*t, back));
  EXPECT(std::equal(norm, norm + 5, back));
}

static void test_header_padding_for_any_name_length(const std::string& root) {
  std::vector<uint16_t> data(64, 0x3c00);
  for (int variant = 0; variant < 5; ++variant) {
    const std::string dir = root + "/v" + std::to_string(variant);
    mkdir(dir.c_str(), 0755);
    {
      SafetensorsWriter wr(dir);
      for (int t = 0; t <= variant; ++t) {
        EXPECT(wr.add("block." + std::to_string(t) + std::string(t + 1, 'x') + ".weight", "F16", {8, 8},
                      data.data(), data.size() * 2));
      }
      EXPECT(wr.close());
    }
    std::ifstream f(dir + "/" + "model-00001-of-00001.safetensors", std::ios::binary);
    uint64_t hlen = 0;
    f.read(reinterpret_cast<char*>(&hlen), 8);
    EXPECT(f.good() && (8 + hlen) % 16 == 0);
  }
}

static void test_config_key_is_merged_into_an_existing_file(const std::string& dir) {
  mkdir(dir.c_str(), 0755);
  {
    std::ofstream f(dir + "/config.json");
    f << "{\n  \"hidden_size\": 4096,\n  \"rope\": {\"theta\": 10000}\n}\n";
  }
  EXPECT(write_quant_config(dir, 64, 4));
  EXPECT(write_quant_config(dir, 32, 8));  // replaced, not duplicated
  std::string text;
  EXPECT(st_detail::read_file(dir + "/config.json", &text));
  EXPECT(text.find("\"hidden_size\": 4096") != std::string::npos);
  EXPECT(text.find("\"quantization\"") == text.rfind("\"quantization\""));
  int g = 0, b = 0;
  EXPECT(read_quant_config(dir, &g, &b) && g == 32 && b == 8);
}

static void test_reader_rejects_damaged_files(const std::string& dir) {
  mkdir(dir.c_str(), 0755);
  SafetensorsReader rd;
  EXPECT(!rd.open_model(dir));  // nothing there
  {
    std::ofstream f(dir + "/model.safetensors", std::ios::binary);
    const std::string hdr = "{\"a\":{\"dtype\":\"F16\",\"shape\":[4],\"data_offsets\":[0,4096]}}";
    const uint64_t n = hdr.size();
    f.write(reinterpret_cast<const char*>(&n), 8);
    f << hdr << "tiny";
  }
  EXPECT(!rd.open_model(dir));  // the range runs past the end of the file
}

int main(int argc, char** argv) {
  const std::string root = argc > 1 ? argv[1] : "/tmp/vpq-safetensors-test";
  mkdir(root.c_str(), 0755);
  test_roundtrip_two_shards(root + "/model");
  test_header_padding_for_any_name_length(root);
  test_config_key_is_merged_into_an_existing_file(root + "/cfg");
  test_reader_rejects_damaged_files(root + "/bad");
  std::printf(g_failed ? "%d FAILED\n" : "ALL PASSED\n", g_failed);
  return g_failed ? 1 : 0;
}
