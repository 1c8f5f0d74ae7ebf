// C++ host side of the MoE path above the C ABI, mirroring the reference's Rust host type for type:
//   check / launched        src/gpu.rs:9-26
//   DevBuf, Stream, Graph   src/gpu.rs:35-163
//   Q8, Q4, Dense           src/model.rs:16-58
//   MoeLayer                the MoE members of src/model.rs:108-121 `Layer`
//   Op, MoeDecoder          src/engine.rs:136-150 (Op), 674-708 (record_step with prefetch chaining),
//                           946-1042 (router_topk + moe_decode per layer, x == res == y), 1047-1066 (step)
// Only dr_* functions from include/dramakernels.h are called: no CUDA headers, no allocation outside dr_malloc.
// The reference's host is Rust; this image has no Rust toolchain, so the same structure is written in C++.
#pragma once

#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/dramakernels.h"

namespace drama {

inline void check(int code, const char* what) {
  if (code != 0) throw std::runtime_error(std::string(what) + ": CUDA error " + std::to_string(code) + " (" + dr_error_string(code) + ")");
}

// Status of a kernel launcher: its own argument check, then the launch error.
inline void launched(int code, const char* what) {
  if (code != 0) throw std::runtime_error(std::string(what) + ": unsupported shape (launcher returned " + std::to_string(code) + ")");
  check(dr_last_error(), what);
}

struct Stream {
  dr_stream raw = nullptr;
  Stream() { check(dr_stream_create(&raw), "stream_create"); }
  ~Stream() {
    if (raw) dr_stream_destroy(raw);
  }
  Stream(const Stream&) = delete;
  Stream& operator=(const Stream&) = delete;
  void sync() const { check(dr_stream_sync(raw), "stream_sync"); }
};

// A device allocation. Pointers handed to kernels stay valid for its lifetime.
class DevBuf {
 public:
  DevBuf() = default;
  explicit DevBuf(size_t bytes) : bytes_(bytes) { check(dr_malloc(&ptr_, bytes ? bytes : 16), "malloc"); }
  DevBuf(const void* host, size_t bytes, const Stream& st) : DevBuf(bytes) {
    check(dr_h2d(ptr_, host, bytes, st.raw), "h2d");
    st.sync();
  }
  static DevBuf zeros(size_t bytes, const Stream& st) {
    DevBuf b(bytes);
    check(dr_memset(b.ptr_, 0, bytes, st.raw), "memset");
    return b;
  }
  DevBuf(DevBuf&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; }
  DevBuf& operator=(DevBuf&& o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_, bytes_ = o.bytes_, o.ptr_ = nullptr;
    }
    return *this;
  }
  DevBuf(const DevBuf&) = delete;
  ~DevBuf() { release(); }
  template <typename T>
  T* ptr() const { return static_cast<T*>(ptr_); }
  template <typename T>
  T* at(size_t elems) const { return static_cast<T*>(ptr_) + elems; }
  size_t bytes() const { return bytes_; }
  void upload(const void* host, size_t n, const Stream& st) const {
    check(dr_h2d(ptr_, host, n, st.raw), "h2d");
    st.sync();
  }
  void download(void* host, size_t n, const Stream& st) const {
    check(dr_d2h(host, ptr_, n, st.raw), "d2h");
    st.sync();
  }

 private:
  void release() {
    if (ptr_) dr_free(ptr_);
    ptr_ = nullptr;
  }
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
};

// Capture `record()` once; replay with launch().
class Graph {
 public:
  Graph(const Stream& st, const std::function<void()>& record) {
    check(dr_graph_begin(st.raw), "graph_begin");
    try {
      record();
    } catch (...) {
      dr_graph_exec tmp = nullptr;
      dr_graph_end(st.raw, &tmp);
      throw;
    }
    check(dr_graph_end(st.raw, &exec_), "graph_end");
  }
  ~Graph() {
    if (exec_) dr_graph_destroy(exec_);
  }
  Graph(const Graph&) = delete;
  void launch(const Stream& st) const { check(dr_graph_launch(exec_, st.raw), "graph_launch"); }

 private:
  dr_graph_exec exec_ = nullptr;
};

// int8 weight, one f16 scale per 128 inputs of a row.
struct Q8 {
  DevBuf q, s;
  size_t n = 0, k = 0;
  std::pair<const int8_t*, const dr_half*> rows(size_t row0) const { return {q.at<int8_t>(row0 * k), s.at<dr_half>(row0 * (k / 128))}; }
};

// Routed experts, int4 asymmetric with group 64: q [E, N, K/2], sm [E, N, K/64, 2].
struct Q4 {
  DevBuf q, sm;
  size_t e = 0, n = 0, k = 0;
  std::pair<const uint8_t*, const dr_half*> expert(size_t ex) const {
    return {q.at<uint8_t>(ex * n * k / 2), sm.at<dr_half>(ex * n * (k / 64) * 2)};
  }
};

struct MoeLayer {
  DevBuf router;     // bf16 [E + 1, H]
  DevBuf post_norm;  // f32 [H]
  Q8 shared_gate_up, shared_down;
  Q4 gate_up, down;
  size_t experts = 0, hidden = 0, inter = 0;
};

// One recorded decode launch. `weights` is the region it streams (for the previous op to prefetch);
// `run` gets the region of the next weight-streaming op to prefetch itself.
struct Op {
  std::optional<std::pair<const char*, size_t>> weights;
  std::function<void(const char*, size_t)> run;
};

constexpr bool ROUTER_PREFETCH = false;  // src/engine.rs:18
constexpr bool GEMV_PREFETCH = true;     // src/engine.rs:19

// Batch-1 decode over a stack of MoE layers: x <- x + moe_l(rmsnorm(x)) for each layer.
class MoeDecoder {
 public:
  MoeDecoder(const std::vector<MoeLayer>& layers, int topk, float eps)
      : layers_(layers), topk_(topk), eps_(eps), hidden_(layers.at(0).hidden) {
    const MoeLayer& l0 = layers.at(0);
    x = DevBuf(hidden_ * 4);
    rlog_ = DevBuf((l0.experts + 1) * 4);
    idx_ = DevBuf(topk * 4);
    wts_ = DevBuf(topk * 4);
    sgate_ = DevBuf(4);
    act_ = DevBuf((topk + 1) * l0.inter * 4);
    counter_ = DevBuf::zeros(16, st);
  }

  std::vector<Op> ops() const {
    std::vector<Op> out;
    for (const MoeLayer& l : layers_) {
      const auto [gq, gs] = l.gate_up.expert(0);
      const auto [dq, ds] = l.down.expert(0);
      const size_t sizes[4] = {l.gate_up.n * l.gate_up.k / 2, l.gate_up.n * (l.gate_up.k / 64) * 4, l.down.n * l.down.k / 2,
                               l.down.n * (l.down.k / 64) * 4};
      const MoeLayer* lp = &l;
      out.push_back(Op{std::make_pair(lp->router.ptr<const char>(), (lp->experts + 1) * lp->hidden * 2),
                       [this, lp, gq = gq, gs = gs, dq = dq, ds = ds, sizes](const char*, size_t) {
                         launched(dr_router_topk(lp->router.ptr<dr_bf16>(), x.ptr<float>(), lp->post_norm.ptr<float>(), eps_,
                                                 rlog_.ptr<float>(), (int)lp->experts, topk_, (int)lp->hidden, idx_.ptr<int>(),
                                                 wts_.ptr<float>(), sgate_.ptr<float>(), counter_.ptr<unsigned>(),
                                                 ROUTER_PREFETCH ? reinterpret_cast<const char*>(gq) : nullptr,
                                                 reinterpret_cast<const char*>(gs), reinterpret_cast<const char*>(dq),
                                                 reinterpret_cast<const char*>(ds), sizes[0], sizes[1], sizes[2], sizes[3], st.raw),
                                  "router_topk");
                       }});
      const auto [sgq, sgs] = l.shared_gate_up.rows(0);
      const auto [sdq, sds] = l.shared_down.rows(0);
      out.push_back(Op{std::nullopt, [this, lp, gq = gq, gs = gs, dq = dq, ds = ds, sgq = sgq, sgs = sgs, sdq = sdq, sds = sds](const char* pf, size_t pfb) {
                         launched(dr_moe_decode(gq, gs, dq, ds, sgq, sgs, sdq, sds, x.ptr<float>(), idx_.ptr<int>(), wts_.ptr<float>(),
                                                sgate_.ptr<float>(), x.ptr<float>(), act_.ptr<float>(), x.ptr<float>(), (int)lp->hidden,
                                                (int)lp->inter, topk_, lp->post_norm.ptr<float>(), eps_, pf, pfb, st.raw),
                                  "moe_decode");
                       }});
    }
    return out;
  }

  // Ops are collected first so every weight-streaming kernel can prefetch the weights of the next one into L2
  // (the last op prefetches the first).
  void record_step() const {
    const std::vector<Op> all = ops();
    std::optional<std::pair<const char*, size_t>> first;
    for (const Op& o : all)
      if (o.weights) {
        first = o.weights;
        break;
      }
    for (size_t k = 0; k < all.size(); ++k) {
      std::optional<std::pair<const char*, size_t>> next;
      for (size_t j = k + 1; j < all.size() && !next; ++j) next = all[j].weights;
      if (!next) next = first;
      if (GEMV_PREFETCH && next) all[k].run(next->first, next->second);
      else all[k].run(nullptr, 0);
    }
  }

  void capture() { graph_ = std::make_unique<Graph>(st, [this] { record_step(); }); }
  void set_x(const float* host) const { x.upload(host, hidden_ * 4, st); }
  // Replays the captured step on the current x and returns the new hidden state.
  std::vector<float> step() const {
    if (!graph_) throw std::runtime_error("capture first");
    graph_->launch(st);
    std::vector<float> y(hidden_);
    x.download(y.data(), hidden_ * 4, st);
    return y;
  }
  std::vector<float> step_eager() const {
    record_step();
    std::vector<float> y(hidden_);
    x.download(y.data(), hidden_ * 4, st);
    return y;
  }
  std::vector<int> routing() const {
    std::vector<int> idx(topk_);
    idx_.download(idx.data(), topk_ * 4, st);
    return idx;
  }

  Stream st;
  DevBuf x;

 private:
  const std::vector<MoeLayer>& layers_;
  int topk_;
  float eps_;
  size_t hidden_;
  DevBuf rlog_, idx_, wts_, sgate_, act_, counter_;
  std::unique_ptr<Graph> graph_;
};

}  // namespace drama
