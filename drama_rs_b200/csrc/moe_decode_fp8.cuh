// Batch-1 MoE decode with block-FP8 routed experts: dr_moe_decode_fp8.
//
// The routed experts are the checkpoint's own E4M3 weights with one f32 scale per 128 x 128 block
// (gate_up: W [E, 2I, H], S [E, 2I/128, H/128]; down: W [E, H, I], S [E, H/128, I/128]); the shared expert stays
// int8. Same two-kernel structure and work split as the int4 path (moe_decode.cuh): 144 gate/up blocks of 32 units,
// >= 128 down blocks of <= 16 rows, all rows of a block requested at once with bulk copies, programmatic dependent
// launch, L2-coherent loads of everything the previous kernel wrote.
//
// Arithmetic: E4M3 has no integer form that dp4a could use, so the routed rows go through
// cvt.rn.f16x2.e4m3x2 (exact), cvt.f32.f16 (exact) and fp32 FMA against fp32 activations, the block scale applied
// once per 16-weight chunk. Measured issue rates on this part: 32 / 155 / 128 per clock and multiprocessor, i.e.
// ~33 weights per clock, against 23 per clock that the HBM rate delivers: the stream stays the bound.
// `act` carries the routed activations as floats ([topk, I], 16 KB) and, behind them, the shared expert's
// activations as 16-value limb blocks (2 KB): exactly the (topk + 1) * I floats of the caller's scratch.
//
// Replaces kernels/drama.cu:602-742 of the reference (fp8x16, dot_fp8, k_moe_gate_up_fp8, k_moe_down_fp8,
// dr_moe_decode_fp8) behind the same C signature (src/ffi.rs:47-51).
#pragma once

#include "moe_decode.cuh"

namespace moe {
namespace f8 {

constexpr int ACT_SHARED_OFF = TOPK * I * 4;  // byte offset of the shared expert's limb blocks in `act`

// Two E4M3 bytes -> two fp16 (low byte -> low half); exact.
DRB_DEV uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t d;
  asm("{.reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t;}" : "=r"(d) : "r"(two_bytes));
  return d;
}

DRB_DEV float2 f16x2_to_f32x2(uint32_t h2) {
  float2 f;
  asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}" : "=f"(f.x), "=f"(f.y) : "r"(h2));
  return f;
}

// sum_k w_k x_k over one 16-byte chunk of E4M3 weights against 16 floats.
DRB_DEV float dot16_fp8(const uint4& v, const float* x) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fl = f16x2_to_f32x2(e4m3x2_to_f16x2(w[i] & 0xffffu)), fh = f16x2_to_f32x2(e4m3x2_to_f16x2(w[i] >> 16));
    a0 = fmaf(fl.x, x[4 * i], a0);
    a1 = fmaf(fl.y, x[4 * i + 1], a1);
    a0 = fmaf(fh.x, x[4 * i + 2], a0);
    a1 = fmaf(fh.y, x[4 * i + 3], a1);
  }
  return a0 + a1;
}

// ------------------------------------------------------------------------------------------
// gate/up

namespace gu8 {

using gu::CW;
using gu::NT;
using gu::QU;
using gu::QUARTERS;
using gu::ROUTED_BLOCKS;
using gu::SSROW;
using gu::THREADS;
using gu::UNITS;
constexpr int GRID = gu::GRID;
constexpr int CTL_BYTES = 1024;
constexpr int XS_BYTES = H * 4;                          // normalised activations: floats (routed blocks) or limb blocks (shared blocks)
constexpr int R_STAGE = 2 * UNITS * H;                   // 131,072: 64 E4M3 rows
constexpr size_t SMEM_BYTES = CTL_BYTES + XS_BYTES + (size_t)gu::S_STAGE;
static_assert(R_STAGE <= gu::S_STAGE && gu::QX_BYTES <= XS_BYTES, "one stage and one activation area serve both kinds of block");

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_gate_up_fp8(const uint8_t* __restrict__ W, const float* __restrict__ S, const int8_t* __restrict__ shq,
                      const __half* __restrict__ shs, const float* __restrict__ x, const int* __restrict__ idx,
                      unsigned char* __restrict__ act, const float* __restrict__ nw, float eps) {
  extern __shared__ __align__(128) unsigned char dyn[];
  gu::Ctl& ctl = *reinterpret_cast<gu::Ctl*>(dyn);
  unsigned char* xs = dyn + CTL_BYTES;
  unsigned char* st = dyn + CTL_BYTES + XS_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x;
  const bool shared = b >= ROUTED_BLOCKS;
  const int slot = b / (I / UNITS);
  const int j0 = shared ? (b - ROUTED_BLOCKS) * UNITS : (b % (I / UNITS)) * UNITS;  // first unit

  if (threadIdx.x == 0) {
    for (int q = 0; q < QUARTERS; ++q) mbar_init(&ctl.full[q], 1);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // ---------------- producer warp: lane 4 q + c requests copy c of part q
    const int q = lane >> 2, c = lane & 3;
    const bool issuing = q < QUARTERS;
    const int u0 = j0 + q * QU, l0 = q * QU;
    if (shared) {
      if (issuing && c == 0) mbar_expect_tx(&ctl.full[q], (unsigned)(2 * QU * (H + SSROW)));
      __syncwarp();
      if (issuing) {
        const unsigned char* sp = reinterpret_cast<const unsigned char*>(shs);
        if (c == 0) bulk_g2s(st + (size_t)l0 * H, shq + (size_t)u0 * H, QU * H, &ctl.full[q]);
        else if (c == 1) bulk_g2s(st + (size_t)(UNITS + l0) * H, shq + ((size_t)I + u0) * H, QU * H, &ctl.full[q]);
        else if (c == 2) bulk_g2s(st + (size_t)2 * UNITS * H + l0 * SSROW, sp + (size_t)u0 * SSROW, QU * SSROW, &ctl.full[q]);
        else bulk_g2s(st + (size_t)2 * UNITS * H + (UNITS + l0) * SSROW, sp + ((size_t)I + u0) * SSROW, QU * SSROW, &ctl.full[q]);
      }
      pdl_wait();
    } else {
      pdl_wait();  // idx is the router's output
      if (issuing && c == 0) mbar_expect_tx(&ctl.full[q], (unsigned)(2 * QU * H));
      __syncwarp();
      if (issuing && c < 2) {
        const uint8_t* wp = W + (size_t)__ldcg(idx + slot) * (2 * I) * H;
        if (c == 0) bulk_g2s(st + (size_t)l0 * H, wp + (size_t)u0 * H, QU * H, &ctl.full[q]);
        else bulk_g2s(st + (size_t)(UNITS + l0) * H, wp + ((size_t)I + u0) * H, QU * H, &ctl.full[q]);
      }
    }
    pdl_launch_dependents();  // never before the wait: the down kernel's prologue reads the router's idx
    return;
  }

  // ---------------- consumers
  const float4 wv = nw ? reinterpret_cast<const float4*>(nw)[threadIdx.x] : make_float4(1.f, 1.f, 1.f, 1.f);
  pdl_wait();               // x is the previous kernel's output
  pdl_launch_dependents();
  const float4 xv = __ldcg(reinterpret_cast<const float4*>(x) + threadIdx.x);
  float inv = 1.f;
  if (nw) {
    const float ss = warp_sum(xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w);
    if (lane == 0) ctl.red[warp] = ss;
    named_sync<NT>();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < CW; ++w) t += ctl.red[w];
    inv = rsqrtf(t / H + eps);
  }
  const float4 xn = make_float4(xv.x * inv * wv.x, xv.y * inv * wv.y, xv.z * inv * wv.z, xv.w * inv * wv.w);
  float v[4];  // v[2i] = gate, v[2i + 1] = up partial sums of this warp's unit warp + 16 i
  if (shared) {
    quant_store_eo(xs, threadIdx.x, xn, true);
    named_sync<NT>();
    QAct<32, true> x0, x1;
    float X0, X1;
    qact_load(x0, X0, xs + (size_t)lane * QB32_BYTES);
    qact_load(x1, X1, xs + (size_t)(32 + lane) * QB32_BYTES);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int u = warp + CW * i;
      mbar_wait(&ctl.full[u / QU], 0, DRB_ERR_FULL_WAIT);
      const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)u * H);
      const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(UNITS + u) * H);
      const __half* gs = reinterpret_cast<const __half*>(st + (size_t)2 * UNITS * H + (size_t)u * SSROW);
      const __half* us = reinterpret_cast<const __half*>(st + (size_t)2 * UNITS * H + (size_t)(UNITS + u) * SSROW);
      v[2 * i] = __half2float(gs[lane >> 2]) * x0.delta * dot32_q8_eo(gr[2 * lane], gr[2 * lane + 1], x0, 0) +
                 __half2float(gs[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(gr[64 + 2 * lane], gr[64 + 2 * lane + 1], x1, 0);
      v[2 * i + 1] = __half2float(us[lane >> 2]) * x0.delta * dot32_q8_eo(ur[2 * lane], ur[2 * lane + 1], x0, 0) +
                     __half2float(us[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(ur[64 + 2 * lane], ur[64 + 2 * lane + 1], x1, 0);
    }
  } else {
    reinterpret_cast<float4*>(xs)[threadIdx.x] = xn;
    named_sync<NT>();
    // This lane owns the 16-byte chunks lane + 32 j (j < 4) of every row: k in [16 (lane + 32 j), +16).
    float xr[4][16];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float4 f = reinterpret_cast<const float4*>(xs)[4 * (lane + 32 * j) + t];
        xr[j][4 * t] = f.x, xr[j][4 * t + 1] = f.y, xr[j][4 * t + 2] = f.z, xr[j][4 * t + 3] = f.w;
      }
    // Block scales: the block's 32 gate rows lie in one 128-row block, so do its up rows; chunk c is k block c / 8.
    const float* se = S + (size_t)__ldcg(idx + slot) * (2 * I / 128) * (H / 128);
    float sg[4], su[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sg[j] = __ldg(se + (size_t)(j0 >> 7) * (H / 128) + (lane >> 3) + 4 * j);
      su[j] = __ldg(se + (size_t)((I + j0) >> 7) * (H / 128) + (lane >> 3) + 4 * j);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int u = warp + CW * i;
      mbar_wait(&ctl.full[u / QU], 0, DRB_ERR_FULL_WAIT);
      const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)u * H);
      const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(UNITS + u) * H);
      float g = 0.f, up = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        g = fmaf(sg[j], dot16_fp8(gr[lane + 32 * j], xr[j]), g);
        up = fmaf(su[j], dot16_fp8(ur[lane + 32 * j], xr[j]), up);
      }
      v[2 * i] = g, v[2 * i + 1] = up;
    }
  }
  // Fold the four per-lane sums into one reduction (as in the int4 kernel).
  const bool hi16 = lane & 16, hi8 = lane & 8;
  const float r0 = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
  const float r1 = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
  float s = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  const float upv = __shfl_xor_sync(0xffffffffu, s, 8);
  if (shared) {
    if ((lane & 15) == 0) ctl.actv[warp + (lane & 16)] = silu_f(s) * upv;
    named_sync<NT>();
    if (warp == 0) gu::quant_block16_halfwarps(ctl.actv[lane], act + ACT_SHARED_OFF + (size_t)(b - ROUTED_BLOCKS) * 2 * QB16_BYTES, lane);
  } else if ((lane & 15) == 0) {
    reinterpret_cast<float*>(act)[slot * I + j0 + warp + (lane & 16)] = silu_f(s) * upv;
  }
}

}  // namespace gu8

// ------------------------------------------------------------------------------------------
// down + combine

namespace dn8 {

using dn::CW;
using dn::NT;
using dn::RT;
using dn::THREADS;
constexpr int MIN_GRID = dn::MIN_GRID;
constexpr int ROW = I;                                        // 512 bytes per E4M3 row
constexpr int STAGE_BYTES = TOPK * RT * ROW + RT * I;         // 65,536 + 8,192 (shared expert, int8)
constexpr int CTL_BYTES = 1024;
constexpr int ACT_BYTES = TOPK * I * 4 + (I / 16) * QB16_BYTES;  // 18,432
constexpr size_t SMEM_BYTES = CTL_BYTES + ACT_BYTES + STAGE_BYTES;
static_assert(ACT_BYTES == (TOPK + 1) * I * 4, "the caller's scratch, byte for byte");

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_down_fp8(const uint8_t* __restrict__ W, const float* __restrict__ S, const int8_t* __restrict__ shq,
                   const __half* __restrict__ shs, const unsigned char* __restrict__ act, const int* __restrict__ idx,
                   const float* __restrict__ wts, const float* __restrict__ sgate, const float* res, float* y,
                   const char* pf, size_t pf_bytes) {
  extern __shared__ __align__(128) unsigned char dyn[];
  dn::Ctl& ctl = *reinterpret_cast<dn::Ctl*>(dyn);
  unsigned char* as = dyn + CTL_BYTES;
  unsigned char* st = as + ACT_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned G = gridDim.x, b = blockIdx.x;
  const int n0 = (int)((long long)H * b / G), n1 = (int)((long long)H * (b + 1) / G);
  const int nr = n1 - n0;  // <= RT because the grid has at least MIN_GRID blocks

  if (threadIdx.x == 0) {
    mbar_init(&ctl.full, 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ---------------- producer warp (launched behind the gate/up kernel, which releases its dependents after its own
    // dependency wait: the routing is final). Lane k < 8 requests expert slot k's rows, lane 8 the shared expert's.
    if (nr > 0) {
      if (lane == 0) mbar_expect_tx(&ctl.full, (unsigned)(nr * (TOPK * ROW + I)));
      __syncwarp();
      if (lane < TOPK) bulk_g2s(st + lane * RT * ROW, W + ((size_t)__ldcg(idx + lane) * H + n0) * ROW, (unsigned)(nr * ROW), &ctl.full);
      else if (lane == TOPK) bulk_g2s(st + TOPK * RT * ROW, shq + (size_t)n0 * I, (unsigned)(nr * I), &ctl.full);
    }
    if (lane == 0) prefetch_share(pf, pf_bytes, b, G);
    return;
  }

  // ---------------- consumers: warp = (expert slot ke, row half rh); the whole warp per row, lane = 16-byte chunk
  const int ke = warp & (TOPK - 1), rh = warp >> 3;
  const float ssc = warp < nr ? __half2float(__ldg(shs + (size_t)(n0 + warp) * (I / 128) + (lane >> 3))) : 0.f;
  // block scales of this warp's rows: constants, fetched before the dependency wait (the routing is final)
  float sc[RT / 2];
  {
    const float* se = S + (size_t)__ldcg(idx + ke) * (H / 128) * (I / 128);
#pragma unroll
    for (int p = 0; p < RT / 2; ++p) {
      const int lr = rh * (RT / 2) + p;
      sc[p] = lr < nr ? __ldg(se + (size_t)((n0 + lr) >> 7) * (I / 128) + (lane >> 3)) : 0.f;
    }
  }
  pdl_wait();  // the activations, and everything the caller wrote before
  {
    // one cooperative copy of the 18 KB of activations (read at L2), with the routing weights
    const uint4* src = reinterpret_cast<const uint4*>(act);
    const uint4 p0 = __ldcg(src + threadIdx.x), p1 = __ldcg(src + NT + threadIdx.x);
    uint4 p2 = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < ACT_BYTES / 16 - 2 * NT) p2 = __ldcg(src + 2 * NT + threadIdx.x);
    float r = 0.f;
    if (threadIdx.x < TOPK) r = __ldcg(wts + threadIdx.x);
    else if (threadIdx.x == TOPK) r = __ldcg(sgate);
    reinterpret_cast<uint4*>(as)[threadIdx.x] = p0;
    reinterpret_cast<uint4*>(as)[NT + threadIdx.x] = p1;
    if (threadIdx.x < ACT_BYTES / 16 - 2 * NT) reinterpret_cast<uint4*>(as)[2 * NT + threadIdx.x] = p2;
    if (threadIdx.x < TOPK) ctl.wk[threadIdx.x] = r;
    else if (threadIdx.x == TOPK) ctl.sgate = r;
  }
  named_sync<NT>();
  float a16[16];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float4 f = reinterpret_cast<const float4*>(as)[(ke * I + 16 * lane) / 4 + t];
    a16[4 * t] = f.x, a16[4 * t + 1] = f.y, a16[4 * t + 2] = f.z, a16[4 * t + 3] = f.w;
  }
  QAct<16, false> sq;
  qact_load(sq, as + ACT_SHARED_OFF + (size_t)lane * QB16_BYTES);
  const float sg = sigmoid_f(ctl.sgate);
  float wk[TOPK];
#pragma unroll
  for (int k = 0; k < TOPK; ++k) wk[k] = ctl.wk[k];

  mbar_wait(&ctl.full, 0, DRB_ERR_FULL_WAIT);
  const unsigned char* eq = st + ke * RT * ROW;
  float v[RT / 2];
#pragma unroll
  for (int p = 0; p < RT / 2; ++p) {
    const int lr = rh * (RT / 2) + p;
    v[p] = 0.f;
    if (lr < nr) v[p] = sc[p] * dot16_fp8(*reinterpret_cast<const uint4*>(eq + (size_t)lr * ROW + 16 * lane), a16);
  }
  {
    // Fold the eight sums (each over all 32 lanes) into one reduction: three exchange steps leave lane group
    // (lane >> 2) with row p = lane >> 2 ... then two butterfly steps finish it.
    static_assert(RT / 2 == 8, "the fold below is written for eight values");
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
    float t4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) t4[i] = (h16 ? v[4 + i] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[4 + i], 16);
    float t2[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) t2[i] = (h8 ? t4[2 + i] : t4[i]) + __shfl_xor_sync(0xffffffffu, h8 ? t4[i] : t4[2 + i], 8);
    float s = (h4 ? t2[1] : t2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? t2[0] : t2[1], 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    const int p = (h16 ? 4 : 0) + (h8 ? 2 : 0) + (h4 ? 1 : 0);
    const int lr = rh * (RT / 2) + p;
    if ((lane & 3) == 0 && lr < nr) ctl.part[ke][lr] = s;
  }
  {
    float s = 0.f;
    if (warp < nr) s = ssc * sq.delta * dot16_q8_i(*reinterpret_cast<const uint4*>(st + TOPK * RT * ROW + (size_t)warp * I + 16 * lane), sq, 0);
    s = warp_sum(s);
    if (lane == 0 && warp < nr) ctl.part[TOPK][warp] = s;
  }
  named_sync<NT>();
  if ((int)threadIdx.x < nr) {
    const int lr = threadIdx.x;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < TOPK; ++k) acc += wk[k] * ctl.part[k][lr];
    y[n0 + lr] = __ldcg(res + n0 + lr) + sg * ctl.part[TOPK][lr] + acc;
  }
}

}  // namespace dn8

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(gu8::k_moe_gate_up_fp8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gu8::SMEM_BYTES)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(dn8::k_moe_down_fp8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dn8::SMEM_BYTES)) != cudaSuccess) return e;
  if ((e = drb_carveout(gu8::k_moe_gate_up_fp8)) != cudaSuccess) return e;
  return drb_carveout(dn8::k_moe_down_fp8);
}

}  // namespace f8
}  // namespace moe

// act must hold (topk + 1) * I floats. x, res and y may be one buffer. Reference: kernels/drama.cu:730-742; src/ffi.rs:47-51.
extern "C" int dr_moe_decode_fp8(const uint8_t* gu_w, const float* gu_s, const uint8_t* d_w, const float* d_s,
                                 const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                                 const float* x, const int* idx, const float* wts, const float* sgate, const float* res,
                                 float* act, float* y, int H, int I, int topk, const float* nw, float eps, const char* pf,
                                 size_t pf_bytes, cudaStream_t st) {
  if (H != moe::H || I != moe::I || topk != moe::TOPK) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  const int g_dn = dev.sms > moe::f8::dn8::MIN_GRID ? dev.sms : moe::f8::dn8::MIN_GRID;
  drb_launch(moe::f8::gu8::k_moe_gate_up_fp8, dim3(moe::f8::gu8::GRID), dim3(moe::f8::gu8::THREADS), moe::f8::gu8::SMEM_BYTES, st,
             dev.pdl, gu_w, gu_s, sgu_q, sgu_s, x, idx, reinterpret_cast<unsigned char*>(act), nw, eps);
  drb_launch(moe::f8::dn8::k_moe_down_fp8, dim3(g_dn), dim3(moe::f8::dn8::THREADS), moe::f8::dn8::SMEM_BYTES, st, dev.pdl, d_w, d_s,
             sd_q, sd_s, reinterpret_cast<const unsigned char*>(act), idx, wts, sgate, res, y, pf, pf_bytes);
  return 0;
}
