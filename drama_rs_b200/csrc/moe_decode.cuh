// Batch-1 MoE decode: dr_moe_decode = gate/up + SwiGLU over the 8 routed int4 experts and the int8
// shared expert, then down projection + weighted combine + sigmoid-gated shared expert + residual.
//
// Both kernels launch at least one block per multiprocessor (148 / 128 blocks at least, so that a
// block's share always fits its shared memory in one go). Every block owns a byte-balanced,
// contiguous share of the weight rows and requests ALL of it at once with bulk asynchronous copies
// (each lane of the producer warp issues the copies of one chunk), so the HBM queue is full from
// the first microsecond. The down kernel is launched with a programmatic dependency: its blocks
// start while gate/up still runs, read the routing, and pull their weight rows into shared memory
// before they wait for the activations.
//
// Activations are read coalesced, normalised, and converted once per block to block fixed point
// (three signed 7-bit limbs per value, see common.cuh); each lane keeps the limb words of its
// k-slice in registers. Weight words then go through dp4a against them: integer-exact sums,
// group scales applied in fp32, warp-shuffle reductions folded over all the rows a warp owns.
//
// Replaces kernels/drama.cu:470-599 of the reference (k_moe_gate_up_q4, k_moe_down_q4,
// dr_moe_decode), behind the same C signature (src/ffi.rs:42-46). Like the reference the launcher
// accepts only H = 2048, I = 512, topk = 8 and returns -1 otherwise.
#pragma once

#include "common.cuh"

namespace moe {

constexpr int H = 2048, I = 512, TOPK = 8;

template <int NT>
DRB_DEV void named_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");
}

// ------------------------------------------------------------------------------------------
// gate/up

namespace gu {

constexpr int CW = 16;                                    // consumer warps, one unit (gate row + up row) at a time each
constexpr int NT = CW * 32;                               // consumer threads
constexpr int THREADS = NT + 32;                          // + one producer warp
constexpr int MIN_GRID = 148;                             // a block then owns <= 28 routed and <= 4 shared units
constexpr int UPW = 2;                                    // units per warp and pass: 32 units over 16 warps
constexpr int RU = 4;                                     // routed units per chunk
constexpr int SU = 2;                                     // shared-expert units per chunk
constexpr int QROW = H / 2;                               // 1024 bytes of nibbles per routed row
constexpr int SMROW = (H / 64) * 4;                       // 128 bytes of (scale, min) per routed row
constexpr int SSROW = (H / 128) * 2;                      // 32 bytes of scales per shared-expert row
constexpr int STAGE_BYTES = RU * 2 * (QROW + SMROW);      // 9216; a shared chunk needs SU*2*(H+32) = 8320
constexpr int STAGES = 12;                                // >= 3 shared + 8 routed chunks (chunks are aligned)
constexpr int CTL_BYTES = 1024;
constexpr int QX_BYTES = (H / 32) * QB32_BYTES;           // the normalised activations as limb blocks
constexpr size_t SMEM_BYTES = CTL_BYTES + QX_BYTES + (size_t)STAGES * STAGE_BYTES;
static_assert(SU * 2 * (H + SSROW) <= STAGE_BYTES, "shared-expert chunk does not fit a stage");
static_assert(NT == H / 4, "one float4 of x per consumer thread");

struct Ctl {
  uint64_t full[STAGES];
  float red[CW];
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
  DRB_DEV int units() const { return (us1 - us0) + (ur1 - ur0); }
  // Units [ua, ub) of chunk t and the aligned base of the chunk. Chunks are aligned to multiples of
  // RU (SU), so a routed chunk never straddles two experts.
  DRB_DEV void chunk(int t, bool& shared, int& base, int& ua, int& ub) const {
    shared = t < nsc;
    if (shared) {
      base = (sc0 + t) * SU, ua = max(base, us0), ub = min(base + SU, us1);
    } else {
      base = (rc0 + t - nsc) * RU, ua = max(base, ur0), ub = min(base + RU, ur1);
    }
  }
  // The o-th unit of the block: shared units first. Returns its chunk and its slot in the chunk.
  DRB_DEV void unit(int o, bool& shared, int& u, int& t, int& slot) const {
    shared = o < us1 - us0;
    if (shared) {
      u = us0 + o, t = u / SU - sc0, slot = u % SU;
    } else {
      u = ur0 + o - (us1 - us0), t = nsc + u / RU - rc0, slot = u % RU;
    }
  }
};

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_gate_up(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
                  const __half* __restrict__ shs, const float* __restrict__ x, const int* __restrict__ idx,
                  float* __restrict__ act, const float* __restrict__ nw, float eps) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* qx = dyn + CTL_BYTES;
  unsigned char* ring = dyn + CTL_BYTES + QX_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Plan plan(blockIdx.x, gridDim.x);
  DRB_TRACE_POINT(10, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&ctl.full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // ---------------- producer warp: lane t requests chunk t
    if (lane < plan.chunks() && lane < STAGES) {
      const int t = lane;
      bool shared;
      int base, ua, ub;
      plan.chunk(t, shared, base, ua, ub);
      unsigned char* dst = ring + (size_t)t * STAGE_BYTES;
      const int n = ub - ua, slot = ua - base;
      if (shared) {
        // The shared expert's rows do not depend on the routing: requested before the dependency wait.
        const unsigned char* sp = reinterpret_cast<const unsigned char*>(shs);
        mbar_expect_tx(&ctl.full[t], (unsigned)(n * 2 * (H + SSROW)));
        bulk_g2s(dst + slot * H, shq + (size_t)ua * H, (unsigned)(n * H), &ctl.full[t]);
        bulk_g2s(dst + (SU + slot) * H, shq + ((size_t)I + ua) * H, (unsigned)(n * H), &ctl.full[t]);
        bulk_g2s(dst + 2 * SU * H + slot * SSROW, sp + (size_t)ua * SSROW, (unsigned)(n * SSROW), &ctl.full[t]);
        bulk_g2s(dst + 2 * SU * H + (SU + slot) * SSROW, sp + ((size_t)I + ua) * SSROW, (unsigned)(n * SSROW), &ctl.full[t]);
      } else {
        pdl_wait();  // idx is the router's output
        DRB_TRACE_POINT(11, CW * 32);
        const int k = ua / I, j = ua % I;
        const size_t ek = (size_t)idx[k];
        const uint8_t* q = Q + ek * (2 * I) * QROW;
        const unsigned char* smp = reinterpret_cast<const unsigned char*>(SM) + ek * (2 * I) * SMROW;
        mbar_expect_tx(&ctl.full[t], (unsigned)(n * 2 * (QROW + SMROW)));
        bulk_g2s(dst + slot * QROW, q + (size_t)j * QROW, (unsigned)(n * QROW), &ctl.full[t]);
        bulk_g2s(dst + (RU + slot) * QROW, q + ((size_t)I + j) * QROW, (unsigned)(n * QROW), &ctl.full[t]);
        bulk_g2s(dst + 2 * RU * QROW + slot * SMROW, smp + (size_t)j * SMROW, (unsigned)(n * SMROW), &ctl.full[t]);
        bulk_g2s(dst + 2 * RU * QROW + (RU + slot) * SMROW, smp + ((size_t)I + j) * SMROW, (unsigned)(n * SMROW), &ctl.full[t]);
      }
    }
    __syncwarp();
    pdl_wait();
    DRB_TRACE_POINT(12, CW * 32);
    pdl_launch_dependents();  // never before the wait: the down kernel's prologue reads the router's idx
    return;
  }

  // ---------------- consumers
  // The norm weight is a constant: fetch it before the dependency wait. Thread t owns float4 t.
  const float4 wv = nw ? reinterpret_cast<const float4*>(nw)[threadIdx.x] : make_float4(1.f, 1.f, 1.f, 1.f);
  pdl_wait();               // x is the previous kernel's output
  pdl_launch_dependents();
  DRB_TRACE_POINT(13, 0);
  const float4 xv = reinterpret_cast<const float4*>(x)[threadIdx.x];
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
  quant_store_eo(qx, threadIdx.x, make_float4(xv.x * inv * wv.x, xv.y * inv * wv.y, xv.z * inv * wv.z, xv.w * inv * wv.w), true);
  named_sync<NT>();
  // This lane owns k in [32 lane, +32) and [1024 + 32 lane, +32): 16-byte chunks lane and 32 + lane of an int4
  // row, chunks {2 lane, 2 lane + 1} and {64 + 2 lane, 64 + 2 lane + 1} of an int8 row.
  QAct<32, true> x0, x1;
  float X0, X1;
  qact_load(x0, X0, qx + (size_t)lane * QB32_BYTES);
  qact_load(x1, X1, qx + (size_t)(32 + lane) * QB32_BYTES);
  DRB_TRACE_POINT(14, 0);

  // Per-lane partial sums of the (up to) UPW units of this warp: v[2i] = gate, v[2i + 1] = up of its i-th unit.
  const int nunits = plan.units();
  for (int o0 = warp; o0 < nunits; o0 += CW * UPW) {
    float v[2 * UPW];
    int uid[UPW];
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const int o = o0 + i * CW;
      v[2 * i] = v[2 * i + 1] = 0.f;
      uid[i] = -1;
      if (o >= nunits) continue;
      bool shared;
      int u, t, slot;
      plan.unit(o, shared, u, t, slot);
      uid[i] = shared ? TOPK * I + u : u;
      const unsigned char* st = ring + (size_t)t * STAGE_BYTES;
      mbar_wait(&ctl.full[t], 0, DRB_ERR_FULL_WAIT);
      if (shared) {
        const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * H);
        const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(SU + slot) * H);
        const __half* gs = reinterpret_cast<const __half*>(st + 2 * SU * H + (size_t)slot * SSROW);
        const __half* us = reinterpret_cast<const __half*>(st + 2 * SU * H + (size_t)(SU + slot) * SSROW);
        v[2 * i] = __half2float(gs[lane >> 2]) * x0.delta * dot32_q8_eo(gr[2 * lane], gr[2 * lane + 1], x0, 0) +
                   __half2float(gs[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(gr[64 + 2 * lane], gr[64 + 2 * lane + 1], x1, 0);
        v[2 * i + 1] = __half2float(us[lane >> 2]) * x0.delta * dot32_q8_eo(ur[2 * lane], ur[2 * lane + 1], x0, 0) +
                       __half2float(us[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(ur[64 + 2 * lane], ur[64 + 2 * lane + 1], x1, 0);
      } else {
        const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * QROW);
        const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(RU + slot) * QROW);
        const __half2* gs = reinterpret_cast<const __half2*>(st + 2 * RU * QROW + (size_t)slot * SMROW);
        const __half2* us = reinterpret_cast<const __half2*>(st + 2 * RU * QROW + (size_t)(RU + slot) * SMROW);
        // w = s*q + m: sum_k w x = s * delta * sum(q n) + m * sum(x) per 64-group; chunk c belongs to group c / 2.
        const float2 g0 = __half22float2(gs[lane >> 1]), g1 = __half22float2(gs[16 + (lane >> 1)]);
        const float2 u0 = __half22float2(us[lane >> 1]), u1 = __half22float2(us[16 + (lane >> 1)]);
        v[2 * i] = g0.x * x0.delta * dot32_q4_i(gr[lane], x0, 0) + g0.y * X0 + g1.x * x1.delta * dot32_q4_i(gr[32 + lane], x1, 0) + g1.y * X1;
        v[2 * i + 1] = u0.x * x0.delta * dot32_q4_i(ur[lane], x0, 0) + u0.y * X0 + u1.x * x1.delta * dot32_q4_i(ur[32 + lane], x1, 0) + u1.y * X1;
      }
    }
    // Fold the four per-lane sums into one reduction: after two exchange steps lane group
    // (lane & 16, lane & 8) carries v[(lane >> 3) & 3]; three butterfly steps finish it.
    static_assert(UPW == 2, "the fold below is written for four values");
    const bool hi16 = lane & 16, hi8 = lane & 8;
    const float r0 = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
    const float r1 = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
    float s = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    // lanes 0..7: gate of unit 0, 8..15: up of unit 0, 16..23: gate of unit 1, 24..31: up of unit 1
    const float upv = __shfl_xor_sync(0xffffffffu, s, 8);
    if ((lane & 15) == 0) {
      const int id = (lane & 16) ? uid[1] : uid[0];
      if (id >= 0) act[id] = silu_f(s) * upv;
    }
  }
  DRB_TRACE_POINT(17, 0);
}

}  // namespace gu

// ------------------------------------------------------------------------------------------
// down + combine

namespace dn {

constexpr int CW = 2 * TOPK;                    // consumer warp w: routed expert slot w & 7, row half w >> 3
constexpr int NT = CW * 32;
constexpr int THREADS = NT + 32;
constexpr int RT = 16;                          // output rows per block at most
constexpr int MIN_GRID = H / RT;                // 128
constexpr int QROW = I / 2;                     // 256 bytes of nibbles per routed row
constexpr int SMROW = (I / 64) * 4;             // 32 bytes of (scale, min)
constexpr int EXPERT_BYTES = RT * (QROW + SMROW);
constexpr int STAGE_BYTES = TOPK * EXPERT_BYTES + RT * I;  // + the shared expert's int8 rows: 45056
constexpr int CTL_BYTES = 1024;
constexpr int QA_BYTES = (TOPK * I / 32) * QB32_BYTES;     // routed activations as even/odd limb blocks
constexpr int QS_BYTES = (I / 16) * QB16_BYTES;            // the shared expert's activations, natural order
constexpr size_t SMEM_BYTES = CTL_BYTES + QA_BYTES + QS_BYTES + STAGE_BYTES;
static_assert(RT == CW, "one shared-expert row per consumer warp");

struct Ctl {
  uint64_t full;
  float part[TOPK + 1][RT];
};

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_down(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
               const __half* __restrict__ shs, const float* __restrict__ act, const int* __restrict__ idx,
               const float* __restrict__ wts, const float* __restrict__ sgate, const float* res, float* y,
               const char* pf, size_t pf_bytes) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* qa = dyn + CTL_BYTES;
  unsigned char* qs = qa + QA_BYTES;
  unsigned char* st = qs + QS_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned G = gridDim.x, b = blockIdx.x;
  const int n0 = (int)((long long)H * b / G), n1 = (int)((long long)H * (b + 1) / G);
  const int nr = n1 - n0;  // <= RT because the grid has at least MIN_GRID blocks
  DRB_TRACE_POINT(20, 0);

  if (threadIdx.x == 0) {
    mbar_init(&ctl.full, 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ---------------- producer warp. This kernel is only ever launched behind k_moe_gate_up, which lets its
    // dependents start after its own dependency wait: the routing is final by the time we get here.
    // Lane k < 8 requests expert slot k's rows, lane 8 the shared expert's.
    if (nr > 0) {
      if (lane == 0) mbar_expect_tx(&ctl.full, (unsigned)(nr * (TOPK * (QROW + SMROW) + I)));
      __syncwarp();
      if (lane < TOPK) {
        const size_t row = (size_t)idx[lane] * H + n0;
        bulk_g2s(st + lane * EXPERT_BYTES, Q + row * QROW, (unsigned)(nr * QROW), &ctl.full);
        bulk_g2s(st + lane * EXPERT_BYTES + RT * QROW, reinterpret_cast<const unsigned char*>(SM) + row * SMROW,
                 (unsigned)(nr * SMROW), &ctl.full);
      } else if (lane == TOPK) {
        bulk_g2s(st + TOPK * EXPERT_BYTES, shq + (size_t)n0 * I, (unsigned)(nr * I), &ctl.full);
      }
    }
    DRB_TRACE_POINT(21, CW * 32);
    if (lane == 0) prefetch_share(pf, pf_bytes, b, G);
    return;
  }

  // ---------------- consumers
  const int ke = warp & (TOPK - 1), rh = warp >> 3;
  // The shared expert's scales are constants: fetched before the dependency wait.
  const float ssc = warp < nr ? __half2float(__ldg(shs + (size_t)(n0 + warp) * (I / 128) + (lane >> 3))) : 0.f;
  pdl_wait();  // act, and everything the caller wrote before
  DRB_TRACE_POINT(22, 0);
  // Quantise the 9 x 512 activations once per block: coalesced reads (all in flight at once).
  constexpr int NR4 = TOPK * I / 4, NS4 = I / 4;  // float4s of the routed part and of the shared part
  constexpr int AV = (NR4 + NS4 + NT - 1) / NT;
  float4 av[AV];
#pragma unroll
  for (int i = 0; i < AV; ++i) {
    const int g = threadIdx.x + i * NT;
    av[i] = g < NR4 + NS4 ? reinterpret_cast<const float4*>(act)[g] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float sg = sigmoid_f(sgate[0]);
  float wk[TOPK];
#pragma unroll
  for (int k = 0; k < TOPK; ++k) wk[k] = wts[k];
#pragma unroll
  for (int i = 0; i < AV; ++i) {
    const int g = threadIdx.x + i * NT;  // a warp's 32 float4s fall on one side of NR4 (both multiples of 32)
    if (g - lane < NR4) quant_store_eo(qa, g, av[i], true);
    else quant_store_nat(qs, g - NR4, av[i], g < NR4 + NS4);
  }
  named_sync<NT>();
  // Half-warps take alternate rows; lane & 15 = 16-byte chunk cc of the row, k in [32 cc, 32 cc + 32).
  const int cc = lane & 15, half = lane >> 4;
  QAct<32, true> aq;
  float A;
  qact_load(aq, A, qa + (size_t)(ke * (I / 32) + cc) * QB32_BYTES);
  QAct<16, false> sq;  // shared expert: the whole warp per row, lane = 16-byte chunk of 16 int8
  qact_load(sq, qs + (size_t)lane * QB16_BYTES);
  DRB_TRACE_POINT(23, 0);

  mbar_wait(&ctl.full, 0, DRB_ERR_FULL_WAIT);
  DRB_TRACE_POINT(24, 0);
  const unsigned char* eq = st + ke * EXPERT_BYTES;
  const unsigned char* esm = eq + RT * QROW;
  // This warp's four row pairs: pass p covers rows 2 (4 rh + p) + half.
  float v[RT / 4];
#pragma unroll
  for (int p = 0; p < RT / 4; ++p) {
    const int lr = 2 * (rh * (RT / 4) + p) + half;
    v[p] = 0.f;
    if (lr < nr) {
      const uint4 w = *reinterpret_cast<const uint4*>(eq + (size_t)lr * QROW + 16 * cc);
      const float2 sm = __half22float2(*reinterpret_cast<const __half2*>(esm + (size_t)lr * SMROW + 4 * (cc >> 1)));
      v[p] = sm.x * aq.delta * dot32_q4_i(w, aq, 0) + sm.y * A;
    }
  }
  {
    // Fold the four sums (each to be reduced over the 16 lanes of a half-warp) into one reduction.
    static_assert(RT / 4 == 4, "the fold below is written for four values");
    const bool hi8 = lane & 8, hi4 = lane & 4;
    const float r0 = (hi8 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi8 ? v[0] : v[2], 8);
    const float r1 = (hi8 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi8 ? v[1] : v[3], 8);
    float s = (hi4 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi4 ? r0 : r1, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    const int p = (hi8 ? 2 : 0) + (hi4 ? 1 : 0);
    const int lr = 2 * (rh * (RT / 4) + p) + half;
    if ((lane & 3) == 0 && lr < nr) ctl.part[ke][lr] = s;
  }
  {
    float s = 0.f;
    if (warp < nr) s = ssc * sq.delta * dot16_q8_i(*reinterpret_cast<const uint4*>(st + TOPK * EXPERT_BYTES + (size_t)warp * I + 16 * lane), sq, 0);
    s = warp_sum(s);
    if (lane == 0 && warp < nr) ctl.part[TOPK][warp] = s;
  }
  named_sync<NT>();
  if ((int)threadIdx.x < nr) {
    const int lr = threadIdx.x;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < TOPK; ++k) acc += wk[k] * ctl.part[k][lr];
    y[n0 + lr] = res[n0 + lr] + sg * ctl.part[TOPK][lr] + acc;
  }
  DRB_TRACE_POINT(25, 0);
}

}  // namespace dn

static cudaError_t configure_all() {
  cudaError_t e = cudaFuncSetAttribute(gu::k_moe_gate_up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gu::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(dn::k_moe_down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dn::SMEM_BYTES)) != cudaSuccess) return e;
  if ((e = drb_carveout(gu::k_moe_gate_up)) != cudaSuccess) return e;
  return drb_carveout(dn::k_moe_down);
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
  const int g_gu = dev.sms > moe::gu::MIN_GRID ? dev.sms : moe::gu::MIN_GRID;
  const int g_dn = dev.sms > moe::dn::MIN_GRID ? dev.sms : moe::dn::MIN_GRID;
  drb_launch(moe::gu::k_moe_gate_up, dim3(g_gu), dim3(moe::gu::THREADS), moe::gu::SMEM_BYTES, st, dev.pdl, gu_q, gu_sm,
             sgu_q, sgu_s, x, idx, act, nw, eps);
  drb_launch(moe::dn::k_moe_down, dim3(g_dn), dim3(moe::dn::THREADS), moe::dn::SMEM_BYTES, st, dev.pdl, d_q, d_sm, sd_q,
             sd_s, (const float*)act, idx, wts, sgate, res, y, pf, pf_bytes);
  return 0;
}
