// dr_moe_decode_static: the batch-1 MoE layer for callers that cannot hand over a scratch buffer.
//
// dr_moe_decode needs (topk + 1) * I floats of scratch between its two kernels and takes them from the
// caller. Some hosts have nothing to give: an engine that sized every byte of device memory for weights and
// caches at start-up and must not grow afterwards, a plugin loaded into a process whose allocator is owned
// by someone else, a helper thread that runs while another thread is capturing a graph and therefore may
// not call cudaMalloc. For them this entry point keeps the scratch inside the library, in a fixed
// file-scope device array. Inputs and outputs are still the caller's.
//
// What follows from that choice:
//  * the array is part of the loaded module: every GPU that loads the library holds its 18 KB until exit;
//  * only the reference shape fits (H = 2048, I = 512, topk = 8, i.e. 4608 floats); anything larger
//    is refused with -1, nothing is silently truncated;
//  * all calls share the one array per device. Two calls that overlap on the GPU (different streams, or a
//    graph replay racing an eager call) overwrite each other's activations. Calls on one stream are safe.
//  * the array keeps the previous call's values; that is harmless here, because the first kernel rewrites
//    every byte that the second kernel reads (16,384 of the 18,432: the activations cross as packed
//    fixed-point blocks, the tail of the array is never touched), so nothing needs clearing.
//
// The first call on a device looks up the array's device address and sets the two kernels' launch
// attributes (no allocation). Make that first call outside any stream capture.
#pragma once

#include "moe_decode.cuh"

namespace moe_static {

constexpr int MAX_SCRATCH_FLOATS = (moe::TOPK + 1) * moe::I;  // 4608 floats = 18 KB

// In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) float g_act_scratch[MAX_SCRATCH_FLOATS];

struct PerDevice {
  float* act;  // device address of g_act_scratch on this device
  int sms;
  bool pdl;
  bool ready;
};
static PerDevice g_dev[32];
static std::mutex g_mu;

// Per-device set-up, with that device current. Nothing here allocates.
static int ensure(int d) {
  std::lock_guard<std::mutex> lock(g_mu);
  PerDevice& pd = g_dev[d];
  if (pd.ready) return 0;
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_act_scratch);
  if (e != cudaSuccess) return (int)e;
  if ((e = moe::configure_all()) != cudaSuccess) return (int)e;
  int sms = 0;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d)) != cudaSuccess) return (int)e;
  const char* v = getenv("DRB_PDL");
  pd.act = static_cast<float*>(p);
  pd.sms = sms;
  pd.pdl = !(v && v[0] == '0');
  pd.ready = true;
  return 0;
}

}  // namespace moe_static

// Same arguments and result as dr_moe_decode without `act`. Returns 0, -1 for a shape whose scratch
// would not fit the built-in array, or a cudaError_t from the one-time set-up.
extern "C" int dr_moe_decode_static(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                                    const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                                    const float* x, const int* idx, const float* wts, const float* sgate,
                                    const float* res, float* y, int H, int I, int topk, const float* nw, float eps,
                                    const char* pf, size_t pf_bytes, cudaStream_t st) {
  if (topk < 1 || I < 1 || (long long)(topk + 1) * I > moe_static::MAX_SCRATCH_FLOATS) return -1;  // scratch would overflow
  if (H != moe::H || I != moe::I || topk != moe::TOPK) return -1;
  int d = 0;
  cudaError_t e = cudaGetDevice(&d);
  if (e != cudaSuccess) return (int)e;
  if (d < 0 || d >= 32) return (int)cudaErrorInvalidDevice;
  const int rc = moe_static::ensure(d);
  if (rc != 0) return rc;
  const moe_static::PerDevice& pd = moe_static::g_dev[d];
  const int g_gu = moe::gu::GRID;
  const int g_dn = pd.sms > moe::dn::MIN_GRID ? pd.sms : moe::dn::MIN_GRID;
  drb_launch(moe::gu::k_moe_gate_up, dim3(g_gu), dim3(moe::gu::THREADS), moe::gu::SMEM_BYTES, st, pd.pdl, gu_q, gu_sm, sgu_q,
             sgu_s, x, idx, reinterpret_cast<unsigned char*>(pd.act), nw, eps);
  drb_launch(moe::dn::k_moe_down, dim3(g_dn), dim3(moe::dn::THREADS), moe::dn::SMEM_BYTES, st, pd.pdl, d_q, d_sm, sd_q, sd_s,
             reinterpret_cast<const unsigned char*>(pd.act), idx, wts, sgate, res, y, pf, pf_bytes);
  return 0;
}
