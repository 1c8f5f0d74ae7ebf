// Batch-1 weight-streaming GEMVs: dr_gemv_q8, dr_gemv_q8_swiglu, dr_gemv_bf16.
//
// One persistent block per multiprocessor owns a contiguous range of output rows. A producer
// thread streams that range through a ring of shared-memory stages with bulk asynchronous copies
// (the whole range is requested at once when it fits the ring); eight or nine consumer warps keep
// their slice of the activation vector in registers, read weight chunks from shared memory as
// 128-bit words, dequantise in registers and reduce with warp shuffles. RMSNorm of the input,
// the residual add, SwiGLU and the L2 prefetch of the next kernel's weights are fused in.
//
// Replaces kernels/drama.cu:219-315 of the reference (k_gemv_q8, k_gemv_q8_swiglu, k_gemv_bf16
// and their launchers), behind the same C signatures (src/ffi.rs:33-40).
#pragma once

#include "common.cuh"

namespace gemv {

constexpr int RING_BYTES = 128 * 1024;
constexpr int MAX_STAGES = 8;

enum Mode { Q8_PLAIN = 0, Q8_SWIGLU = 1, BF16_PLAIN = 2 };

struct Smem {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  float red[64];      // cross-warp partials (K split over several warps, or the norm's sum of squares)
  float inv_rms;
};

// Named barrier over the consumer warps only (the producer warp never joins).
DRB_DEV void consumer_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }

// KSEG: elements of K one warp covers (512 or 2048). NSEG: warps that share a row (K = KSEG * NSEG).
// RPW: rows a warp handles per stage. CW: consumer warps.
template <int KSEG, int NSEG, int RPW, int CW, int MODE>
__global__ void __launch_bounds__((CW + 1) * 32, 1)
    k_gemv(const void* __restrict__ Wv, const __half* __restrict__ S, const float* __restrict__ x, const float* res,
           float* y, int N, const float* __restrict__ nw, float eps, const char* pf, size_t pf_bytes) {
  constexpr int K = KSEG * NSEG;
  constexpr int ESZ = MODE == BF16_PLAIN ? 2 : 1;            // bytes per weight
  constexpr int EPC = 16 / ESZ;                              // weights per 16-byte chunk
  constexpr int NCH = KSEG / EPC / 32;                       // chunks per lane per row segment
  constexpr int U = MODE == Q8_SWIGLU ? 2 : 1;               // weight rows per output
  constexpr int RG = CW / NSEG;                              // rows in flight per pass
  constexpr int RB = RG * RPW;                               // outputs per stage
  constexpr int ROW_BYTES = K * ESZ;
  constexpr int SROW = MODE == BF16_PLAIN ? 0 : (K / 128) * 2;  // bytes of group scales per weight row
  constexpr bool S_IN_STAGE = SROW >= 16;                     // bulk copies need 16-byte granules
  constexpr int STAGE_BYTES = RB * U * (ROW_BYTES + (S_IN_STAGE ? SROW : 0));
  constexpr int STAGES = RING_BYTES / STAGE_BYTES < MAX_STAGES ? RING_BYTES / STAGE_BYTES : MAX_STAGES;
  constexpr int NT = CW * 32;
  static_assert(STAGES >= 2, "ring too small");
  static_assert(NCH >= 1, "segment too small");

  extern __shared__ __align__(128) unsigned char dyn[];
  Smem& sm = *reinterpret_cast<Smem*>(dyn);
  float4* xs4 = reinterpret_cast<float4*>(dyn + 1024);
  unsigned char* ring = dyn + 1024 + K * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned G = gridDim.x, b = blockIdx.x;
  const int u0 = (int)((long long)N * b / G), u1 = (int)((long long)N * (b + 1) / G);
  const int nchunks = (u1 - u0 + RB - 1) / RB;
  const unsigned char* W = reinterpret_cast<const unsigned char*>(Wv);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], CW);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ---------------- producer: weights are constants, so copies start before the dependency wait
    if (lane == 0) {
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % STAGES;
        if (c >= STAGES && !mbar_wait(&sm.empty[s], ((c / STAGES) - 1) & 1, DRB_ERR_EMPTY_WAIT)) break;
        const int r0 = u0 + c * RB;
        const int nr = min(RB, u1 - r0);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&sm.full[s], (unsigned)(nr * U * (ROW_BYTES + (S_IN_STAGE ? SROW : 0))));
        bulk_g2s(dst, W + (size_t)r0 * ROW_BYTES, (unsigned)(nr * ROW_BYTES), &sm.full[s]);
        if (U == 2) bulk_g2s(dst + RB * ROW_BYTES, W + ((size_t)N + r0) * ROW_BYTES, (unsigned)(nr * ROW_BYTES), &sm.full[s]);
        if (S_IN_STAGE) {
          const unsigned char* sp = reinterpret_cast<const unsigned char*>(S);
          unsigned char* sd = dst + U * RB * ROW_BYTES;
          bulk_g2s(sd, sp + (size_t)r0 * SROW, (unsigned)(nr * SROW), &sm.full[s]);
          if (U == 2) bulk_g2s(sd + RB * SROW, sp + ((size_t)N + r0) * SROW, (unsigned)(nr * SROW), &sm.full[s]);
        }
      }
      prefetch_share(pf, pf_bytes, b, G);
    }
    return;
  }

  // ---------------- consumers
  pdl_wait();  // x and res come from the previous kernel
  const int seg = warp % NSEG, rg = warp / NSEG;
  float inv = 1.f;
  if (nw) {
    float ss = 0.f;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = threadIdx.x; i < K / 4; i += NT) {
      const float4 v = __ldcg(x4 + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) sm.red[32 + warp] = ss;
    consumer_sync(NT);
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < CW; ++w) t += sm.red[32 + w];
    inv = rsqrtf(t / K + eps);
  }
  // Stage the (normalised) activations once per block: coalesced read, then either a swizzled float4 store
  // (bf16 weights keep fp32 activations) or conversion to limb blocks of 16 values (int8 weights, dp4a).
  // Chunk c = lane + 32*i of the segment covers k = seg*KSEG + EPC*c ...; whole warps enter or skip the loop.
  unsigned char* qb = reinterpret_cast<unsigned char*>(xs4);
  for (int i = threadIdx.x; i < K / 4; i += NT) {
    float4 v = __ldcg(reinterpret_cast<const float4*>(x) + i);
    if (nw) {
      const float4 w = reinterpret_cast<const float4*>(nw)[i];
      v = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w);
    }
    if (MODE == BF16_PLAIN) xs4[swz4(i)] = v;
    else quant_store_nat(qb, i, v, true);
  }
  consumer_sync(NT);
  unsigned long long xp[MODE == BF16_PLAIN ? NCH * EPC / 2 : 1];
  QAct<16, false> xq[MODE == BF16_PLAIN ? 1 : NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    if (MODE == BF16_PLAIN) {
      const int g0 = (seg * KSEG + EPC * (lane + 32 * i)) / 4;
#pragma unroll
      for (int e = 0; e < EPC / 4; ++e) {
        const float4 v = xs4[swz4(g0 + e)];
        xp[i * (EPC / 2) + 2 * e] = pack2(v.x, v.y);
        xp[i * (EPC / 2) + 2 * e + 1] = pack2(v.z, v.w);
      }
    } else {
      qact_load(xq[i], qb + (size_t)(seg * (KSEG / 16) + lane + 32 * i) * QB16_BYTES);
    }
  }

  bool dead = false;
  for (int c = 0; c < nchunks; ++c) {
    const int s = c % STAGES;
    const int r0 = u0 + c * RB;
    const int nr = min(RB, u1 - r0);
    const unsigned char* st = ring + (size_t)s * STAGE_BYTES;
    // Group scales come straight from global memory; issue them before waiting on the copy.
    float sc[RPW][U][NCH];
    if (MODE != BF16_PLAIN) {
#pragma unroll
      for (int p = 0; p < RPW; ++p) {
        const int lr = p * RG + rg;
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < NCH; ++i) {
            const size_t row = (size_t)(u ? N : 0) + r0 + lr;
            sc[p][u][i] = (!S_IN_STAGE && lr < nr) ? __half2float(__ldg(S + row * (K / 128) + (seg * KSEG + 16 * (lane + 32 * i)) / 128)) : 0.f;
          }
      }
    }
    // after the first wait of this thread that ran out no later wait spins again: the error word is set, the
    // results are void, and a vocabulary-sized launch must not hold the GPU for a second per remaining chunk
    if (!dead) dead = !mbar_wait(&sm.full[s], (c / STAGES) & 1, DRB_ERR_FULL_WAIT);
    if (MODE != BF16_PLAIN && S_IN_STAGE) {
      const __half* ss = reinterpret_cast<const __half*>(st + U * RB * ROW_BYTES);
#pragma unroll
      for (int p = 0; p < RPW; ++p) {
        const int lr = p * RG + rg;
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < NCH; ++i)
            sc[p][u][i] = lr < nr ? __half2float(ss[(u * RB + lr) * (K / 128) + (seg * KSEG + 16 * (lane + 32 * i)) / 128]) : 0.f;
      }
    }
#pragma unroll
    for (int p = 0; p < RPW; ++p) {
      const int lr = p * RG + rg;
      float d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        d[u] = 0.f;
        if (lr < nr) {
          const unsigned char* rowp = st + (size_t)(u * RB + lr) * ROW_BYTES + (size_t)seg * KSEG * ESZ;
          if (MODE == BF16_PLAIN) {
            unsigned long long a0 = 0ull, a1 = 0ull;
#pragma unroll
            for (int i = 0; i < NCH; i += 2) {
              a0 = dot8_bf16(*reinterpret_cast<const uint4*>(rowp + 16 * (lane + 32 * i)), xp + i * 4, a0);
              if (i + 1 < NCH) a1 = dot8_bf16(*reinterpret_cast<const uint4*>(rowp + 16 * (lane + 32 * (i + 1))), xp + (i + 1) * 4, a1);
            }
            float p0, p1, p2, p3;
            unpack2(a0, p0, p1);
            unpack2(a1, p2, p3);
            d[u] = (p0 + p1) + (p2 + p3);
          } else {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
              d[u] += sc[p][u][i] * xq[i].delta * dot16_q8_i(*reinterpret_cast<const uint4*>(rowp + 16 * (lane + 32 * i)), xq[i], 0);
          }
        }
        d[u] = warp_sum(d[u]);
      }
      if (NSEG == 1) {
        if (lane == 0 && lr < nr) {
          const int row = r0 + lr;
          y[row] = U == 2 ? silu_f(d[0]) * d[U - 1] : d[0] + (res ? __ldcg(res + row) : 0.f);
        }
      } else {
        // K is split over NSEG warps: combine their partial sums in segment order.
        if (lane == 0) {
          sm.red[(rg * NSEG + seg) * 2] = d[0];
          sm.red[(rg * NSEG + seg) * 2 + 1] = d[U - 1];
        }
        consumer_sync(CW * 32);
        if (seg == 0 && lane == 0 && lr < nr) {
          float t0 = 0.f, t1 = 0.f;
#pragma unroll
          for (int q = 0; q < NSEG; ++q) {
            t0 += sm.red[(rg * NSEG + q) * 2];
            t1 += sm.red[(rg * NSEG + q) * 2 + 1];
          }
          const int row = r0 + lr;
          y[row] = U == 2 ? silu_f(t0) * t1 : t0 + (res ? __ldcg(res + row) : 0.f);
        }
        consumer_sync(CW * 32);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);
  }
}

template <int KSEG, int NSEG, int RPW, int CW, int MODE>
constexpr size_t smem_bytes() {
  constexpr int K = KSEG * NSEG;
  constexpr int ESZ = MODE == BF16_PLAIN ? 2 : 1;
  constexpr int U = MODE == Q8_SWIGLU ? 2 : 1;
  constexpr int SROW = MODE == BF16_PLAIN ? 0 : (K / 128) * 2;
  constexpr int STAGE = (CW / NSEG) * RPW * U * (K * ESZ + (SROW >= 16 ? SROW : 0));
  constexpr int STAGES = RING_BYTES / STAGE < MAX_STAGES ? RING_BYTES / STAGE : MAX_STAGES;
  return 1024 + (size_t)K * 4 + (size_t)STAGES * STAGE;
}

template <int KSEG, int NSEG, int RPW, int CW, int MODE>
int launch(const void* W, const __half* S, const float* x, const float* res, float* y, int N, const float* nw, float eps,
           const char* pf, size_t pf_bytes, cudaStream_t st) {
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (N <= 0) return 0;
  const int grid = N < dev.sms ? N : dev.sms;
  auto kern = k_gemv<KSEG, NSEG, RPW, CW, MODE>;
  drb_launch(kern, dim3(grid), dim3((CW + 1) * 32), smem_bytes<KSEG, NSEG, RPW, CW, MODE>(), st, dev.pdl, W, S, x, res, y, N,
             nw, eps, pf, pf_bytes);
  return 0;
}

template <int KSEG, int NSEG, int RPW, int CW, int MODE>
cudaError_t configure() {
  cudaError_t e = cudaFuncSetAttribute(k_gemv<KSEG, NSEG, RPW, CW, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem_bytes<KSEG, NSEG, RPW, CW, MODE>());
  if (e != cudaSuccess) return e;
  return drb_carveout(k_gemv<KSEG, NSEG, RPW, CW, MODE>);
}

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = configure<512, 1, 4, 8, Q8_PLAIN>()) != cudaSuccess) return e;
  if ((e = configure<2048, 1, 1, 8, Q8_PLAIN>()) != cudaSuccess) return e;
  if ((e = configure<2048, 2, 1, 8, Q8_PLAIN>()) != cudaSuccess) return e;
  if ((e = configure<2048, 3, 1, 9, Q8_PLAIN>()) != cudaSuccess) return e;
  if ((e = configure<2048, 4, 1, 8, Q8_PLAIN>()) != cudaSuccess) return e;
  if ((e = configure<2048, 1, 1, 8, Q8_SWIGLU>()) != cudaSuccess) return e;
  if ((e = configure<2048, 2, 1, 8, Q8_SWIGLU>()) != cudaSuccess) return e;
  if ((e = configure<2048, 1, 1, 8, BF16_PLAIN>()) != cudaSuccess) return e;
  return cudaSuccess;
}

}  // namespace gemv

// y[n] = W[n] . rmsnorm?(x) (+ res[n]); y may alias res. K in {512, 2048, 4096, 6144, 8192}, else -1.
// Reference: kernels/drama.cu:283-294; src/ffi.rs:33-36.
extern "C" int dr_gemv_q8(const int8_t* W, const __half* S, const float* x, const float* res, float* y, int N, int K,
                          const float* nw, float eps, const char* pf, size_t pf_bytes, cudaStream_t st) {
  using namespace gemv;
  switch (K) {
    case 512: return launch<512, 1, 4, 8, Q8_PLAIN>(W, S, x, res, y, N, nw, eps, pf, pf_bytes, st);
    case 2048: return launch<2048, 1, 1, 8, Q8_PLAIN>(W, S, x, res, y, N, nw, eps, pf, pf_bytes, st);
    case 4096: return launch<2048, 2, 1, 8, Q8_PLAIN>(W, S, x, res, y, N, nw, eps, pf, pf_bytes, st);
    case 6144: return launch<2048, 3, 1, 9, Q8_PLAIN>(W, S, x, res, y, N, nw, eps, pf, pf_bytes, st);
    case 8192: return launch<2048, 4, 1, 8, Q8_PLAIN>(W, S, x, res, y, N, nw, eps, pf, pf_bytes, st);
    default: return -1;
  }
}

// y[j] = silu(W[j] . x) * (W[I + j] . x), W is [2I, K]. K in {2048, 4096}, else -1.
// Reference: kernels/drama.cu:296-305; src/ffi.rs:37-39.
extern "C" int dr_gemv_q8_swiglu(const int8_t* W, const __half* S, const float* x, float* y, int I, int K, const float* nw,
                                 float eps, const char* pf, size_t pf_bytes, cudaStream_t st) {
  using namespace gemv;
  switch (K) {
    case 2048: return launch<2048, 1, 1, 8, Q8_SWIGLU>(W, S, x, nullptr, y, I, nw, eps, pf, pf_bytes, st);
    case 4096: return launch<2048, 2, 1, 8, Q8_SWIGLU>(W, S, x, nullptr, y, I, nw, eps, pf, pf_bytes, st);
    default: return -1;
  }
}

// y[n] = W[n] . rmsnorm?(x) for bf16 weights. K == 2048, else -1.
// Reference: kernels/drama.cu:307-315; src/ffi.rs:40.
extern "C" int dr_gemv_bf16(const __nv_bfloat16* W, const float* x, float* y, int N, int K, const float* nw, float eps,
                            const char* pf, size_t pf_bytes, cudaStream_t st) {
  using namespace gemv;
  if (K != 2048) return -1;
  return launch<2048, 1, 1, 8, BF16_PLAIN>(W, nullptr, x, nullptr, y, N, nw, eps, pf, pf_bytes, st);
}
