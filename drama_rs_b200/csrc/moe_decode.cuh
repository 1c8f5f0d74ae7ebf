// Batch-1 MoE decode: dr_moe_decode = gate/up + SwiGLU over the 8 routed int4 experts and the int8
// shared expert, then down projection + weighted combine + sigmoid-gated shared expert + residual.
//
// Both kernels run one persistent block per multiprocessor. Every block owns a byte-balanced,
// contiguous share of the weight rows and requests ALL of it at once with bulk asynchronous copies
// into shared memory (the shares are ~80 KB and ~40 KB), so the HBM queue is full from the first
// microsecond. The down kernel is launched with a programmatic dependency: its blocks start while
// gate/up still runs, read the routing, and pull their weight rows into shared memory before they
// wait for the activations. Consumer warps hold their slice of the activations in registers and
// dequantise in registers (see common.cuh).
//
// Replaces kernels/drama.cu:470-599 of the reference (k_moe_gate_up_q4, k_moe_down_q4,
// dr_moe_decode), behind the same C signature (src/ffi.rs:42-46). Like the reference the launcher
// accepts only H = 2048, I = 512, topk = 8 and returns -1 otherwise.
#pragma once

#include "common.cuh"

namespace moe {

constexpr int H = 2048, I = 512, TOPK = 8;
constexpr int CW = 8;                  // consumer warps
constexpr int THREADS = (CW + 1) * 32;  // + one producer warp

DRB_DEV void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory"); }

// Sum of squares of x[0..2048) over the consumer warps -> rsqrt(mean + eps). red: 8 floats + 1.
DRB_DEV float rms_scale(const float* __restrict__ x, float eps, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < H / 4 / (CW * 32); ++i) {
    const float4 v = x4[threadIdx.x + i * CW * 32];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  consumer_sync();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < CW; ++w) t += red[w];
    red[CW] = rsqrtf(t / H + eps);
  }
  consumer_sync();
  return red[CW];
}

// ------------------------------------------------------------------------------------------
// gate/up

namespace gu {

constexpr int RU = 4;                                     // routed units (gate row + up row) per chunk
constexpr int SU = 2;                                     // shared-expert units per chunk
constexpr int QROW = H / 2;                               // 1024 bytes of nibbles per routed row
constexpr int SMROW = (H / 64) * 4;                       // 128 bytes of (scale, min) per routed row
constexpr int STAGE_BYTES = RU * 2 * (QROW + SMROW);      // 9216; a shared chunk needs SU*2*H = 8192
constexpr int STAGES = 12;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES;

struct Ctl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  float red[CW + 1];
};

struct Plan {
  int us0, us1, ur0, ur1;  // this block's shared units and routed units
  int sc0, nsc, rc0, nrc;  // aligned chunk ranges
  DRB_DEV Plan(unsigned b, unsigned G) {
    us0 = (int)((long long)I * b / G), us1 = (int)((long long)I * (b + 1) / G);
    ur0 = (int)((long long)TOPK * I * b / G), ur1 = (int)((long long)TOPK * I * (b + 1) / G);
    sc0 = us0 / SU, nsc = us1 > us0 ? (us1 + SU - 1) / SU - sc0 : 0;
    rc0 = ur0 / RU, nrc = ur1 > ur0 ? (ur1 + RU - 1) / RU - rc0 : 0;
  }
  DRB_DEV int chunks() const { return nsc + nrc; }
  // Units [ua, ub) of chunk t, the aligned base of the chunk, and whether it is a shared-expert chunk.
  DRB_DEV void chunk(int t, bool& shared, int& base, int& ua, int& ub) const {
    shared = t < nsc;
    if (shared) {
      base = (sc0 + t) * SU, ua = max(base, us0), ub = min(base + SU, us1);
    } else {
      base = (rc0 + t - nsc) * RU, ua = max(base, ur0), ub = min(base + RU, ur1);
    }
  }
  DRB_DEV int ordinal(bool shared, int u) const { return shared ? u - us0 : (us1 - us0) + (u - ur0); }
};

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_gate_up(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
                  const __half* __restrict__ shs, const float* __restrict__ x, const int* __restrict__ idx,
                  float* __restrict__ act, const float* __restrict__ nw, float eps) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* ring = dyn + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Plan plan(blockIdx.x, gridDim.x);
  const int T = plan.chunks();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], CW);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // ---------------- producer
    if (lane == 0) {
      int e[TOPK];
      bool have_idx = false;
      for (int t = 0; t < T; ++t) {
        const int s = t % STAGES;
        if (t >= STAGES && !mbar_wait(&ctl.empty[s], ((t / STAGES) - 1) & 1, DRB_ERR_EMPTY_WAIT)) break;
        bool shared;
        int base, ua, ub;
        plan.chunk(t, shared, base, ua, ub);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        const int n = ub - ua, slot = ua - base;
        if (shared) {
          // The shared expert's rows do not depend on the routing: requested before the dependency wait.
          mbar_expect_tx(&ctl.full[s], (unsigned)(n * 2 * H));
          bulk_g2s(dst + slot * H, shq + (size_t)ua * H, (unsigned)(n * H), &ctl.full[s]);
          bulk_g2s(dst + (SU + slot) * H, shq + ((size_t)I + ua) * H, (unsigned)(n * H), &ctl.full[s]);
        } else {
          if (!have_idx) {
            pdl_wait();  // idx is the router's output
#pragma unroll
            for (int k = 0; k < TOPK; ++k) e[k] = idx[k];
            have_idx = true;
          }
          const int k = ua / I, j = ua % I;
          int ek = e[0];
#pragma unroll
          for (int q = 1; q < TOPK; ++q) ek = k == q ? e[q] : ek;
          const uint8_t* q = Q + (size_t)ek * (2 * I) * QROW;
          const unsigned char* smp = reinterpret_cast<const unsigned char*>(SM) + (size_t)ek * (2 * I) * SMROW;
          mbar_expect_tx(&ctl.full[s], (unsigned)(n * 2 * (QROW + SMROW)));
          bulk_g2s(dst + slot * QROW, q + (size_t)j * QROW, (unsigned)(n * QROW), &ctl.full[s]);
          bulk_g2s(dst + (RU + slot) * QROW, q + ((size_t)I + j) * QROW, (unsigned)(n * QROW), &ctl.full[s]);
          bulk_g2s(dst + 2 * RU * QROW + slot * SMROW, smp + (size_t)j * SMROW, (unsigned)(n * SMROW), &ctl.full[s]);
          bulk_g2s(dst + 2 * RU * QROW + (RU + slot) * SMROW, smp + ((size_t)I + j) * SMROW, (unsigned)(n * SMROW), &ctl.full[s]);
        }
      }
      if (!have_idx) pdl_wait();
    }
    __syncwarp();
    pdl_launch_dependents();
    return;
  }

  // ---------------- consumers
  pdl_wait();               // x is the previous kernel's output
  pdl_launch_dependents();  // only now: the down kernel's prologue reads the router's idx
  const float inv = nw ? rms_scale(x, eps, ctl.red) : 1.f;
  // This lane owns k in [32*lane, 32*lane + 32) and [1024 + 32*lane, 1024 + 32*lane + 32).
  unsigned long long xp[32];
  float X[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int k0 = h * 1024 + 32 * lane;
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float4 v = *reinterpret_cast<const float4*>(x + k0 + 4 * e);
      if (nw) {
        const float4 w = *reinterpret_cast<const float4*>(nw + k0 + 4 * e);
        v = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w);
      }
      xp[h * 16 + 2 * e] = pack2(v.x, v.y);
      xp[h * 16 + 2 * e + 1] = pack2(v.z, v.w);
      sum += (v.x + v.y) + (v.z + v.w);
    }
    X[h] = sum;
  }

  for (int t = 0; t < T; ++t) {
    const int s = t % STAGES;
    bool shared;
    int base, ua, ub;
    plan.chunk(t, shared, base, ua, ub);
    const unsigned char* st = ring + (size_t)s * STAGE_BYTES;
    bool waited = false;
    for (int u = ua; u < ub; ++u) {
      if ((plan.ordinal(shared, u) & (CW - 1)) != warp) continue;
      const int slot = u - base;
      float g, up;
      if (shared) {
        // int8 rows: this lane's k ranges are the 16-byte chunks {2l, 2l+1} and {64+2l, 64+2l+1}.
        const float sg0 = __half2float(__ldg(shs + (size_t)u * (H / 128) + (lane >> 2)));
        const float sg1 = __half2float(__ldg(shs + (size_t)u * (H / 128) + 8 + (lane >> 2)));
        const float su0 = __half2float(__ldg(shs + ((size_t)I + u) * (H / 128) + (lane >> 2)));
        const float su1 = __half2float(__ldg(shs + ((size_t)I + u) * (H / 128) + 8 + (lane >> 2)));
        if (!waited) mbar_wait(&ctl.full[s], (t / STAGES) & 1, DRB_ERR_FULL_WAIT), waited = true;
        const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * H);
        const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(SU + slot) * H);
        g = sg0 * (dot16_q8(gr[2 * lane], xp) + dot16_q8(gr[2 * lane + 1], xp + 8)) +
            sg1 * (dot16_q8(gr[64 + 2 * lane], xp + 16) + dot16_q8(gr[64 + 2 * lane + 1], xp + 24));
        up = su0 * (dot16_q8(ur[2 * lane], xp) + dot16_q8(ur[2 * lane + 1], xp + 8)) +
             su1 * (dot16_q8(ur[64 + 2 * lane], xp + 16) + dot16_q8(ur[64 + 2 * lane + 1], xp + 24));
      } else {
        if (!waited) mbar_wait(&ctl.full[s], (t / STAGES) & 1, DRB_ERR_FULL_WAIT), waited = true;
        const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * QROW);
        const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(RU + slot) * QROW);
        const __half2* gs = reinterpret_cast<const __half2*>(st + 2 * RU * QROW + (size_t)slot * SMROW);
        const __half2* us = reinterpret_cast<const __half2*>(st + 2 * RU * QROW + (size_t)(RU + slot) * SMROW);
        // chunk c = lane and lane + 32; group = c / 2. w = s*q + m and the dots carry a +16 offset per
        // weight, so the group's constant term is (m - 16 s) * sum(x).
        const float2 g0 = __half22float2(gs[lane >> 1]), g1 = __half22float2(gs[16 + (lane >> 1)]);
        const float2 u0 = __half22float2(us[lane >> 1]), u1 = __half22float2(us[16 + (lane >> 1)]);
        g = g0.x * dot32_q4(gr[lane], xp) + (g0.y - 16.f * g0.x) * X[0] + g1.x * dot32_q4(gr[32 + lane], xp + 16) +
            (g1.y - 16.f * g1.x) * X[1];
        up = u0.x * dot32_q4(ur[lane], xp) + (u0.y - 16.f * u0.x) * X[0] + u1.x * dot32_q4(ur[32 + lane], xp + 16) +
             (u1.y - 16.f * u1.x) * X[1];
      }
      g = warp_sum(g);
      up = warp_sum(up);
      if (lane == 0) act[shared ? TOPK * I + u : u] = silu_f(g) * up;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ctl.empty[s]);
  }
}

}  // namespace gu

// ------------------------------------------------------------------------------------------
// down + combine

namespace dn {

constexpr int RT = 16;                          // output rows per tile
constexpr int QROW = I / 2;                     // 256 bytes of nibbles per routed row
constexpr int SMROW = (I / 64) * 4;             // 32 bytes of (scale, min)
constexpr int EXPERT_BYTES = RT * (QROW + SMROW);
constexpr int STAGE_BYTES = TOPK * EXPERT_BYTES + RT * I;  // + the shared expert's int8 rows: 45056
constexpr int STAGES = 2;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES;

struct Ctl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  float part[TOPK + 1][RT];
};

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_down(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
               const __half* __restrict__ shs, const float* __restrict__ act, const int* __restrict__ idx,
               const float* __restrict__ wts, const float* __restrict__ sgate, const float* res, float* y,
               const char* pf, size_t pf_bytes) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* ring = dyn + 1024;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned G = gridDim.x, b = blockIdx.x;
  const int n0 = (int)((long long)H * b / G), n1 = (int)((long long)H * (b + 1) / G);
  const int T = (n1 - n0 + RT - 1) / RT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], CW);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ---------------- producer. This kernel is only ever launched behind k_moe_gate_up, which lets its
    // dependents start after its own dependency wait: the routing is final by the time we get here.
    if (lane == 0) {
      for (int t = 0; t < T; ++t) {
        const int s = t % STAGES;
        if (t >= STAGES && !mbar_wait(&ctl.empty[s], ((t / STAGES) - 1) & 1, DRB_ERR_EMPTY_WAIT)) break;
        const int r0 = n0 + t * RT, nr = min(RT, n1 - r0);
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&ctl.full[s], (unsigned)(nr * (TOPK * (QROW + SMROW) + I)));
        for (int k = 0; k < TOPK; ++k) {
          const size_t row = (size_t)idx[k] * H + r0;
          bulk_g2s(dst + k * EXPERT_BYTES, Q + row * QROW, (unsigned)(nr * QROW), &ctl.full[s]);
          bulk_g2s(dst + k * EXPERT_BYTES + RT * QROW, reinterpret_cast<const unsigned char*>(SM) + row * SMROW,
                   (unsigned)(nr * SMROW), &ctl.full[s]);
        }
        bulk_g2s(dst + TOPK * EXPERT_BYTES, shq + (size_t)r0 * I, (unsigned)(nr * I), &ctl.full[s]);
      }
      prefetch_share(pf, pf_bytes, b, G);
    }
    return;
  }

  // ---------------- consumers: warp k owns routed expert slot k
  pdl_wait();  // act, and everything the caller wrote before
  // Half-warps take alternate rows; lane & 15 = 16-byte chunk cc of the row, k in [32 cc, 32 cc + 32).
  const int cc = lane & 15, half = lane >> 4;
  unsigned long long ap[16];
  float A = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float4 v = *reinterpret_cast<const float4*>(act + warp * I + 32 * cc + 4 * e);
    ap[2 * e] = pack2(v.x, v.y), ap[2 * e + 1] = pack2(v.z, v.w);
    A += (v.x + v.y) + (v.z + v.w);
  }
  // Shared expert: the whole warp per row, lane = 16-byte chunk of 16 int8.
  unsigned long long sp[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float4 v = *reinterpret_cast<const float4*>(act + TOPK * I + 16 * lane + 4 * e);
    sp[2 * e] = pack2(v.x, v.y), sp[2 * e + 1] = pack2(v.z, v.w);
  }
  const float sg = sigmoid_f(sgate[0]);

  for (int t = 0; t < T; ++t) {
    const int s = t % STAGES;
    const int r0 = n0 + t * RT, nr = min(RT, n1 - r0);
    const unsigned char* st = ring + (size_t)s * STAGE_BYTES;
    float ssc[RT / CW];
#pragma unroll
    for (int p = 0; p < RT / CW; ++p) {
      const int lr = p * CW + warp;
      ssc[p] = lr < nr ? __half2float(__ldg(shs + (size_t)(r0 + lr) * (I / 128) + (lane >> 3))) : 0.f;
    }
    mbar_wait(&ctl.full[s], (t / STAGES) & 1, DRB_ERR_FULL_WAIT);
    const unsigned char* eq = st + warp * EXPERT_BYTES;
    const unsigned char* esm = eq + RT * QROW;
#pragma unroll
    for (int p = 0; p < RT / 2; ++p) {
      const int lr = 2 * p + half;
      float v = 0.f;
      if (lr < nr) {
        const uint4 w = *reinterpret_cast<const uint4*>(eq + (size_t)lr * QROW + 16 * cc);
        const float2 sm = __half22float2(*reinterpret_cast<const __half2*>(esm + (size_t)lr * SMROW + 4 * (cc >> 1)));
        v = sm.x * dot32_q4(w, ap) + (sm.y - 16.f * sm.x) * A;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (cc == 0 && lr < nr) ctl.part[warp][lr] = v;
    }
#pragma unroll
    for (int p = 0; p < RT / CW; ++p) {
      const int lr = p * CW + warp;
      float v = 0.f;
      if (lr < nr) v = ssc[p] * dot16_q8(*reinterpret_cast<const uint4*>(st + TOPK * EXPERT_BYTES + (size_t)lr * I + 16 * lane), sp);
      v = warp_sum(v);
      if (lane == 0 && lr < nr) ctl.part[TOPK][lr] = v;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ctl.empty[s]);
    consumer_sync();
    if ((int)threadIdx.x < nr) {
      const int lr = threadIdx.x;
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < TOPK; ++k) acc += wts[k] * ctl.part[k][lr];
      y[r0 + lr] = res[r0 + lr] + sg * ctl.part[TOPK][lr] + acc;
    }
    consumer_sync();
  }
}

}  // namespace dn

static cudaError_t configure_all() {
  cudaError_t e = cudaFuncSetAttribute(gu::k_moe_gate_up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gu::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(dn::k_moe_down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dn::SMEM_BYTES);
}

}  // namespace moe

// act must hold (topk + 1) * I floats. x, res and y may be one buffer (the reference's caller passes the
// same pointer three times): every read of x happens in the first kernel, every write of y in the second.
// Reference: kernels/drama.cu:588-599; src/ffi.rs:42-46.
extern "C" int dr_moe_decode(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                             const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                             const float* x, const int* idx, const float* wts, const float* sgate, const float* res,
                             float* act, float* y, int H, int I, int topk, const float* nw, float eps, const char* pf,
                             size_t pf_bytes, cudaStream_t st) {
  if (H != moe::H || I != moe::I || topk != moe::TOPK) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  drb_launch(moe::gu::k_moe_gate_up, dim3(dev.sms), dim3(moe::THREADS), moe::gu::SMEM_BYTES, st, dev.pdl, gu_q, gu_sm, sgu_q,
             sgu_s, x, idx, act, nw, eps);
  drb_launch(moe::dn::k_moe_down, dim3(dev.sms), dim3(moe::THREADS), moe::dn::SMEM_BYTES, st, dev.pdl, d_q, d_sm, sd_q, sd_s,
             (const float*)act, idx, wts, sgate, res, y, pf, pf_bytes);
  return 0;
}
