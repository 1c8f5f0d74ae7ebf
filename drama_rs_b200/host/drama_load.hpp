// Reads the MoE tensors of one `layerNN.safetensors` of a drama-rs-v1 checkpoint and uploads them.
// Mirrors src/model.rs:217-227 (the keys a layer loads) and src/model.rs:60-105 (dtype / shape checks on load).
// The safetensors container: u64 little-endian header length, a JSON object
//   {"name": {"dtype": "..", "shape": [..], "data_offsets": [begin, end]}, ...}, then the raw bytes.
#pragma once

#include <cstdio>
#include <fstream>
#include <map>

#include "drama_host.hpp"

namespace drama {

constexpr const char* LAYER_TENSORS[] = {"moe.router",          "post_norm",      "moe.shared_gate_up.q8", "moe.shared_gate_up.s",
                                         "moe.shared_down.q8",  "moe.shared_down.s", "moe.gate_up.q4",      "moe.gate_up.sm",
                                         "moe.down.q4",         "moe.down.sm"};

struct TensorInfo {
  std::string dtype;
  std::vector<size_t> shape;
  size_t begin = 0, end = 0;
};

inline size_t dtype_bytes(const std::string& dtype) {
  if (dtype == "U8" || dtype == "I8" || dtype == "BOOL" || dtype == "F8_E4M3" || dtype == "F8_E5M2") return 1;
  if (dtype == "F16" || dtype == "BF16" || dtype == "I16" || dtype == "U16") return 2;
  if (dtype == "F32" || dtype == "I32" || dtype == "U32") return 4;
  if (dtype == "F64" || dtype == "I64" || dtype == "U64") return 8;
  return 0;
}

// Every tensor of the header is validated before anything is read: its byte range must lie inside the file, in order,
// and be exactly as long as its shape and dtype say. A truncated or malformed file is refused here, on the host; what
// reaches the device always has the size the kernels assume.
class SafeTensors {
 public:
  explicit SafeTensors(const std::string& path) : path_(path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + path);
    const uint64_t file_size = (uint64_t)f.tellg();
    f.seekg(0);
    uint64_t n = 0;
    f.read(reinterpret_cast<char*>(&n), 8);
    if (!f || n == 0 || n > (1u << 26) || 8 + n > file_size) throw std::runtime_error(path + ": bad safetensors header length");
    std::string js(n, '\0');
    f.read(js.data(), (std::streamsize)n);
    if (!f) throw std::runtime_error(path + ": truncated header");
    data0_ = 8 + n;
    parse(js);
    const uint64_t data_bytes = file_size - data0_;
    for (const auto& kv : tensors_) {
      const TensorInfo& t = kv.second;
      const size_t esz = dtype_bytes(t.dtype);
      if (esz == 0) throw std::runtime_error(path + ": " + kv.first + ": unknown dtype " + t.dtype);
      uint64_t count = 1;
      for (size_t d : t.shape) {
        if (d != 0 && count > (uint64_t(1) << 48) / d) throw std::runtime_error(path + ": " + kv.first + ": shape overflows");
        count *= d;
      }
      if (t.begin > t.end || t.end > data_bytes) throw std::runtime_error(path + ": " + kv.first + ": data range outside the file (truncated?)");
      if (t.end - t.begin != count * esz) throw std::runtime_error(path + ": " + kv.first + ": data size does not match shape and dtype");
    }
  }

  const TensorInfo& info(const std::string& name) const {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) throw std::runtime_error(path_ + ": missing tensor " + name);
    return it->second;
  }

  std::vector<char> read(const std::string& name) const {
    const TensorInfo& t = info(name);
    std::vector<char> out(t.end - t.begin);
    std::ifstream f(path_, std::ios::binary);
    f.seekg((std::streamoff)(data0_ + t.begin));
    f.read(out.data(), (std::streamsize)out.size());
    if (!f) throw std::runtime_error(path_ + ": truncated data for " + name);
    return out;
  }

 private:
  // The header is flat enough for a hand scanner: top-level keys map to objects with three known members.
  // Every access is bounded: running off the end of the header is a parse error, never a read past the string.
  void parse(const std::string& s) {
    size_t p = 0;
    auto fail = [&]() -> void { throw std::runtime_error(path_ + ": header parse error"); };
    auto at = [&]() -> char {
      if (p >= s.size()) fail();
      return s[p];
    };
    auto skip = [&] { while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r' || s[p] == ',' || s[p] == ':')) ++p; };
    auto str = [&] {
      if (at() != '"') fail();
      const size_t q = ++p;
      while (at() != '"') {
        p += (s[p] == '\\') ? 2 : 1;
        if (p > s.size()) fail();
      }
      std::string out = s.substr(q, p - q);
      ++p;
      return out;
    };
    auto numbers = [&] {
      std::vector<size_t> out;
      if (at() != '[') fail();
      ++p;
      for (;;) {
        skip();
        if (at() == ']') { ++p; return out; }
        if (s[p] < '0' || s[p] > '9') fail();
        size_t v = 0;
        while (p < s.size() && s[p] >= '0' && s[p] <= '9') {
          if (v > (~size_t(0) - 9) / 10) fail();
          v = v * 10 + (size_t)(s[p++] - '0');
        }
        out.push_back(v);
      }
    };
    skip();
    if (at() != '{') fail();
    ++p;
    for (;;) {
      skip();
      if (p >= s.size() || s[p] == '}') return;
      const std::string name = str();
      skip();
      if (at() != '{') fail();
      ++p;
      TensorInfo t;
      for (;;) {
        skip();
        if (at() == '}') { ++p; break; }
        const std::string key = str();
        skip();
        if (key == "dtype") t.dtype = str();
        else if (key == "shape") t.shape = numbers();
        else if (key == "data_offsets") {
          auto v = numbers();
          if (v.size() != 2) fail();
          t.begin = v[0], t.end = v[1];
        }
        else if (at() == '"') str();  // "__metadata__": {"k": "v"}
        else throw std::runtime_error(path_ + ": unexpected header member " + key);
      }
      if (name != "__metadata__") tensors_[name] = std::move(t);
    }
  }

  std::string path_;
  size_t data0_ = 0;
  std::map<std::string, TensorInfo> tensors_;
};

// CRC-32 (IEEE, reflected) of a tensor's bytes: what `--inspect` prints so that a host-side check can compare values.
inline uint32_t crc32_bytes(const std::vector<char>& v) {
  uint32_t c = 0xFFFFFFFFu;
  for (char ch : v) {
    c ^= (uint8_t)ch;
    for (int k = 0; k < 8; ++k) c = (c >> 1) ^ (0xEDB88320u & (0u - (c & 1u)));
  }
  return ~c;
}

inline DevBuf upload_checked(const SafeTensors& f, const std::string& name, const char* dtype, const std::vector<size_t>& shape,
                             const Stream& st) {
  const TensorInfo& t = f.info(name);
  if (t.dtype != dtype) throw std::runtime_error(name + ": dtype " + t.dtype + ", expected " + dtype);
  if (t.shape != shape) throw std::runtime_error(name + ": unexpected shape");
  const std::vector<char> bytes = f.read(name);
  return DevBuf(bytes.data(), bytes.size(), st);
}

// The geometry comes from moe.gate_up.q4 [E, 2I, H/2]; every other tensor is checked against it.
inline MoeLayer load_moe_layer(const std::string& path, const Stream& st) {
  SafeTensors f(path);
  const std::vector<size_t>& g = f.info("moe.gate_up.q4").shape;
  if (g.size() != 3) throw std::runtime_error("moe.gate_up.q4: expected rank 3");
  const size_t e = g[0], i = g[1] / 2, h = g[2] * 2;
  MoeLayer l;
  l.experts = e, l.hidden = h, l.inter = i;
  l.router = upload_checked(f, "moe.router", "BF16", {e + 1, h}, st);
  l.post_norm = upload_checked(f, "post_norm", "F32", {h}, st);
  l.shared_gate_up = Q8{upload_checked(f, "moe.shared_gate_up.q8", "I8", {2 * i, h}, st),
                        upload_checked(f, "moe.shared_gate_up.s", "F16", {2 * i, h / 128}, st), 2 * i, h};
  l.shared_down = Q8{upload_checked(f, "moe.shared_down.q8", "I8", {h, i}, st),
                     upload_checked(f, "moe.shared_down.s", "F16", {h, i / 128}, st), h, i};
  l.gate_up = Q4{upload_checked(f, "moe.gate_up.q4", "U8", {e, 2 * i, h / 2}, st),
                 upload_checked(f, "moe.gate_up.sm", "F16", {e, 2 * i, h / 64, 2}, st), e, 2 * i, h};
  l.down = Q4{upload_checked(f, "moe.down.q4", "U8", {e, h, i / 2}, st), upload_checked(f, "moe.down.sm", "F16", {e, h, i / 64, 2}, st), e,
              h, i};
  return l;
}

}  // namespace drama
