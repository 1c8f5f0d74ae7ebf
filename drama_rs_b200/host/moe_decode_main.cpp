// Command-line driver of the C++ host: batch-1 decode through a stack of MoE layers.
//   moe_decode_main --inspect layer00.safetensors      (no GPU: prints the MoE tensors' dtypes, shapes, sizes and CRC-32s)
//   moe_decode_main --x x.f32 --out-eager a.f32 --out-graph b.f32 [--steps N] [--topk 8] [--eps 1e-6] layer00.safetensors ...
// Runs one eager step from x, then captures the step and replays it `steps` times from x again; writes the hidden
// state after the eager step and after the last replay, and prints the per-step time of the replays.
#include <chrono>
#include <cstdlib>
#include <iostream>

#include "drama_load.hpp"

static std::vector<float> read_f32(const std::string& path) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) throw std::runtime_error("cannot open " + path);
  const size_t n = (size_t)f.tellg();
  std::vector<float> v(n / 4);
  f.seekg(0);
  f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)n);
  return v;
}

static void write_f32(const std::string& path, const std::vector<float>& v) {
  std::ofstream f(path, std::ios::binary);
  f.write(reinterpret_cast<const char*>(v.data()), (std::streamsize)(v.size() * 4));
  if (!f) throw std::runtime_error("cannot write " + path);
}

int main(int argc, char** argv) try {
  std::string xp, eager_out, graph_out;
  int steps = 1, topk = 8;
  float eps = 1e-6f;
  std::vector<std::string> files;
  for (int a = 1; a < argc; ++a) {
    const std::string s = argv[a];
    auto val = [&] {
      if (a + 1 >= argc) throw std::runtime_error("missing value after " + s);
      return std::string(argv[++a]);
    };
    if (s == "--inspect") {
      const drama::SafeTensors f(val());
      for (const char* name : drama::LAYER_TENSORS) {
        const drama::TensorInfo& t = f.info(name);
        std::cout << name << " " << t.dtype;
        for (size_t d : t.shape) std::cout << " " << d;
        std::cout << " bytes=" << (t.end - t.begin) << " crc32=" << drama::crc32_bytes(f.read(name)) << "\n";
      }
      return 0;
    }
    if (s == "--x") xp = val();
    else if (s == "--out-eager") eager_out = val();
    else if (s == "--out-graph") graph_out = val();
    else if (s == "--steps") steps = std::atoi(val().c_str());
    else if (s == "--topk") topk = std::atoi(val().c_str());
    else if (s == "--eps") eps = (float)std::atof(val().c_str());
    else files.push_back(s);
  }
  if (xp.empty() || files.empty()) {
    std::cerr << "usage: moe_decode_main --x x.f32 [--out-eager f] [--out-graph f] [--steps n] [--topk k] [--eps e] layer.safetensors...\n";
    return 2;
  }
  drama::check(drb_init(), "init");
  std::vector<drama::MoeLayer> layers;
  {
    drama::Stream up;
    for (const std::string& f : files) layers.push_back(drama::load_moe_layer(f, up));
  }
  const std::vector<float> x = read_f32(xp);
  if (x.size() != layers[0].hidden) throw std::runtime_error("x has the wrong length");

  drama::MoeDecoder dec(layers, topk, eps);
  dec.set_x(x.data());
  const std::vector<float> eager = dec.step_eager();
  if (!eager_out.empty()) write_f32(eager_out, eager);

  dec.capture();
  dec.set_x(x.data());
  std::vector<float> y;
  const auto t0 = std::chrono::steady_clock::now();
  for (int s = 0; s < steps; ++s) y = dec.step();
  const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / steps;
  if (!graph_out.empty()) write_f32(graph_out, y);
  unsigned err = 0;
  drama::check(drb_device_error(&err), "device_error");
  std::cout << "{\"layers\": " << layers.size() << ", \"steps\": " << steps << ", \"us_per_step_host_clock\": " << us
            << ", \"device_error\": " << err << "}\n";
  return err ? 1 : 0;
} catch (const std::exception& e) {
  std::cerr << "moe_decode_main: " << e.what() << "\n";
  return 1;
}
