// Runtime wrappers of the C ABI (allocation, copies, streams, graph capture, cuBLAS) and the
// per-device setup the kernels need before their first launch.
//
// Mirrors kernels/drama.cu:1991-2044 of the reference (src/ffi.rs:13-31). The reference's host calls
// dr_stream_create, dr_cublas_create and dr_sample_init before it captures its decode graph
// (src/engine.rs:168-170, 332-335); those hooks (and dr_malloc) run the device setup here, so that the
// launchers, whose first call happens inside the capture, never have to allocate or set attributes.
#pragma once

#include <cublas_v2.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

// Every kernel of the library asks for the same shared-memory carveout (the maximum). Kernels that
// prefer different L1/shared splits cannot share a multiprocessor, and switching the split between
// consecutive launches drains it first: microseconds per launch on a path whose kernels run for two.
template <typename K>
static cudaError_t drb_carveout(K kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

namespace gemv { static cudaError_t configure_all(); }
namespace router { static cudaError_t configure_all(); }
namespace pf { static cudaError_t configure_all(); }
namespace moe { static cudaError_t configure_all(); namespace f8 { static cudaError_t configure_all(); } }
namespace stack { static cudaError_t configure_all(); }
namespace pfmma { static cudaError_t configure_all(); }
namespace pft { static cudaError_t configure_all(); }
namespace pf8 { static cudaError_t configure_all(); }

namespace rt {

constexpr int MAX_DEVICES = 32;
static DrbDevice g_dev[MAX_DEVICES];
static std::atomic<bool> g_ready[MAX_DEVICES];  // g_dev[d] is complete (release / acquire)
static const DrbDevice g_unready = {};
static std::mutex g_mu;
static cudaError_t g_setup_error = cudaSuccess;

static cudaError_t setup(int d) {
  DrbDevice dv = {};
  cudaError_t e;
  int sms = 0;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d)) != cudaSuccess) return e;
  dv.sms = sms;
  const char* p = getenv("DRB_PDL");
  dv.pdl = !(p && p[0] == '0');
  if ((e = gemv::configure_all()) != cudaSuccess) return e;
  if ((e = router::configure_all()) != cudaSuccess) return e;
  if ((e = pf::configure_all()) != cudaSuccess) return e;
  if ((e = moe::configure_all()) != cudaSuccess) return e;
  if ((e = moe::f8::configure_all()) != cudaSuccess) return e;
  if ((e = stack::configure_all()) != cudaSuccess) return e;
  if ((e = pfmma::configure_all()) != cudaSuccess) return e;
  if ((e = pft::configure_all()) != cudaSuccess) return e;
  if ((e = pf8::configure_all()) != cudaSuccess) return e;
  dv.ready = true;
  g_dev[d] = dv;
  g_ready[d].store(true, std::memory_order_release);
  return cudaSuccess;
}

// Runs the setup for the current device if it has not run yet. Must not be called while the calling
// thread captures a stream (it allocates).
static cudaError_t ensure() {
  int d = 0;
  cudaError_t e = cudaGetDevice(&d);
  if (e != cudaSuccess) return e;
  if (d < 0 || d >= MAX_DEVICES) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_ready[d].load(std::memory_order_acquire)) return cudaSuccess;
  e = setup(d);
  g_setup_error = e;
  return e;
}

}  // namespace rt

const DrbDevice& drb_device(cudaStream_t st) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= rt::MAX_DEVICES) return rt::g_unready;
  if (rt::g_ready[d].load(std::memory_order_acquire)) return rt::g_dev[d];
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return rt::g_unready;
  if (rt::ensure() != cudaSuccess) return rt::g_unready;
  return rt::g_dev[d];
}

#define DRB_API extern "C"

DRB_API int dr_last_error(void) { return (int)cudaGetLastError(); }
DRB_API const char* dr_error_string(int e) { return cudaGetErrorString((cudaError_t)e); }
DRB_API int dr_malloc(void** p, size_t n) {
  rt::ensure();
  return (int)cudaMalloc(p, n);
}
DRB_API int dr_free(void* p) { return (int)cudaFree(p); }
DRB_API int dr_host_alloc(void** p, size_t n) { return (int)cudaMallocHost(p, n); }
DRB_API int dr_host_free(void* p) { return (int)cudaFreeHost(p); }
DRB_API int dr_h2d(void* d, const void* h, size_t n, cudaStream_t st) {
  return (int)cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, st);
}
DRB_API int dr_d2h(void* h, const void* d, size_t n, cudaStream_t st) {
  return (int)cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, st);
}
DRB_API int dr_d2d(void* d, const void* s, size_t n, cudaStream_t st) {
  return (int)cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, st);
}
DRB_API int dr_memset(void* d, int v, size_t n, cudaStream_t st) { return (int)cudaMemsetAsync(d, v, n, st); }
DRB_API int dr_stream_create(cudaStream_t* s) {
  const cudaError_t e = rt::ensure();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamCreateWithFlags(s, cudaStreamNonBlocking);
}
DRB_API int dr_stream_destroy(cudaStream_t s) { return (int)cudaStreamDestroy(s); }
DRB_API int dr_stream_sync(cudaStream_t s) { return (int)cudaStreamSynchronize(s); }
DRB_API int dr_device_sync(void) { return (int)cudaDeviceSynchronize(); }
DRB_API int dr_mem_info(size_t* free_b, size_t* total_b) { return (int)cudaMemGetInfo(free_b, total_b); }

// Capture is thread-local, as in the reference (kernels/drama.cu:2018), so another thread driving its
// own stream does not break it.
DRB_API int dr_graph_begin(cudaStream_t s) { return (int)cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal); }
DRB_API int dr_graph_end(cudaStream_t s, cudaGraphExec_t* exec) {
  cudaGraph_t g;
  cudaError_t e = cudaStreamEndCapture(s, &g);
  if (e != cudaSuccess) return (int)e;
  e = cudaGraphInstantiate(exec, g, 0);
  cudaGraphDestroy(g);
  return (int)e;
}
DRB_API int dr_graph_launch(cudaGraphExec_t exec, cudaStream_t s) { return (int)cudaGraphLaunch(exec, s); }
DRB_API int dr_graph_destroy(cudaGraphExec_t exec) { return (int)cudaGraphExecDestroy(exec); }

DRB_API int dr_cublas_create(void** h, cudaStream_t s) {
  rt::ensure();
  cublasHandle_t handle;
  cublasStatus_t r = cublasCreate(&handle);
  if (r != CUBLAS_STATUS_SUCCESS) return (int)r;
  r = cublasSetStream(handle, s);
  *h = handle;
  return (int)r;
}
DRB_API int dr_cublas_destroy(void* h) { return (int)cublasDestroy((cublasHandle_t)h); }

// C[M, N] (row-major, f32) = A[M, K] (bf16) . W[N, K]^T (bf16) + beta * C. A plain library GEMM, as in the
// reference (kernels/drama.cu:2040-2044): the prefill router logits and the shared expert go through it.
DRB_API int dr_gemm(void* h, const __nv_bfloat16* A, const __nv_bfloat16* W, float* C, int M, int N, int K, float beta) {
  const float alpha = 1.f;
  return (int)cublasGemmEx((cublasHandle_t)h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, W, CUDA_R_16BF, K, A, CUDA_R_16BF, K,
                           &beta, C, CUDA_R_32F, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
}

// The reference's sampling setup hook (src/ffi.rs:105); sampling is outside this library, but the hook is
// one of the calls the host makes before capture, so it runs the device setup.
DRB_API int dr_sample_init(void) { return (int)rt::ensure(); }

// ---- additions of this library (no counterpart in the reference's ABI) -------------------------------

// Explicit device setup for hosts that want to do it themselves; 0 or a cudaError_t.
DRB_API int drb_init(void) { return (int)rt::ensure(); }

// Reads and clears the error word that bounded device-side waits set when they give up
// (0 = none; see DrbError). Synchronises the device.
DRB_API int drb_device_error(unsigned* out) {
  unsigned zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_drb_error, sizeof(unsigned));
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyToSymbol(g_drb_error, &zero, sizeof(unsigned));
}

// Blocks the persistent kernels launch on the current device (the multiprocessor count).
DRB_API int drb_grid_blocks(void) {
  if (rt::ensure() != cudaSuccess) return -1;
  int d = 0;
  cudaGetDevice(&d);
  return rt::g_dev[d].sms;
}
