// drb_moe_stack_decode: a whole stack of MoE layers at batch 1 in ONE persistent kernel.
//
//   for each layer:  x <- x + moe_l(rmsnorm(x, post_norm_l))
//
// This is the 40-layer decode step of the benchmark (hidden state carried layer to layer) without
// the 120 kernel boundaries of the per-layer calls. It has no counterpart in the reference's ABI
// (there the token mixer sits between two MoE blocks); the per-layer entry points dr_router_topk and
// dr_moe_decode remain the drop-in path and compute the same thing.
//
// One block per multiprocessor, launched cooperatively (all blocks resident). A layer has four phases
// separated by three grid-wide barriers:
//   P0  every block normalises and quantises x; blocks 0..128 compute two router logits each
//   --- barrier: logits complete
//   P1  every block reads the 257 logits and derives the top-8 itself (identical everywhere); its
//       producer warp then requests its share of the chosen experts' gate/up rows AND down rows
//   P2  gate/up + SwiGLU on the block's share -> act
//   --- barrier: act complete
//   P3  down + combine on the block's 13-14 output rows -> x
//   --- barrier: x complete
// Weights that do not depend on the routing (router rows, shared expert) are requested one phase to
// one layer ahead, so they are in shared memory when needed. The code stays hot in the instruction
// cache across layers, nothing is relaunched, and x / act / logits cross blocks through L2 only.
//
// Every grid barrier is a bounded spin on a counter in global memory; when a wait runs out the
// kernel sets the device error word, stops waiting anywhere else, and runs to its end.
#pragma once

#include <cooperative_groups.h>

#include "moe_decode.cuh"
#include "router.cuh"

// One layer's weights, device pointers in the reference's layouts (see include/dramakernels.h).
struct drb_moe_layer {
  const void* router;     // bf16 [E + 1, 2048]
  const void* post_norm;  // f32 [2048]
  const void* gu_q;       // u8  [E, 1024, 1024]
  const void* gu_sm;      // f16 [E, 1024, 32, 2]
  const void* d_q;        // u8  [E, 2048, 256]
  const void* d_sm;       // f16 [E, 2048, 8, 2]
  const void* sgu_q;      // i8  [1024, 2048]
  const void* sgu_s;      // f16 [1024, 16]
  const void* sd_q;       // i8  [2048, 512]
  const void* sd_s;       // f16 [2048, 4]
};

namespace stack {

using moe::H;
using moe::I;
using moe::TOPK;

// The persistent kernel keeps its own work split for the gate/up phase (byte-balanced shares of units, cut into
// chunks that travel through a ring of stages) and quantises the activations per block in the down phase.
namespace gu1 {
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
}  // namespace gu1
namespace dn1 {
constexpr int QA_BYTES = (TOPK * I / 32) * QB32_BYTES;  // routed activations as even/odd limb blocks
constexpr int QS_BYTES = (I / 16) * QB16_BYTES;         // the shared expert's activations, natural order
}  // namespace dn1


namespace dn = moe::dn;

constexpr int CW = 16;
constexpr int NT = CW * 32;
constexpr int THREADS = NT + 32;
constexpr int MAX_E = 256;

// Workspace in global memory (caller-provided, see drb_moe_stack_workspace_bytes).
constexpr int MAX_BLOCKS = 256;
struct Workspace {
  unsigned flags[MAX_BLOCKS];  // flags[0] counts barrier arrivals; zeroed before every launch
  float logits[MAX_E + 8];
  float act[(TOPK + 1) * I];
};

// Shared memory map.
constexpr int CTL_BYTES = 4096;
constexpr int XS_BYTES = H * 4;                          // normalised x in fp32 (router dot)
constexpr int QX_BYTES = gu1::QX_BYTES;                   // normalised x as limb blocks
constexpr int RW_BYTES = 2 * 2 * H * 2;                  // two router rows, double-buffered over layers
constexpr int QA_BYTES = dn1::QA_BYTES + dn1::QS_BYTES;    // act as limb blocks
constexpr int RING_BYTES = gu1::STAGES * gu1::STAGE_BYTES; // gate/up chunks
constexpr int DST_BYTES = dn::STAGE_BYTES;               // down rows
constexpr size_t SMEM_BYTES = CTL_BYTES + XS_BYTES + QX_BYTES + RW_BYTES + QA_BYTES + RING_BYTES + DST_BYTES;

struct Ctl {
  uint64_t gfull[gu1::STAGES];  // one phase per layer each
  uint64_t dfull_routed, dfull_shared;
  uint64_t rfull[2];           // router rows of even / odd layers
  float red[CW];
  float part[TOPK + 1][dn::RT];
  float rpart[2][8];
  int idx[TOPK];
  float wts[TOPK];
  float sgate;
  int abort;                   // set once a grid barrier timed out: no further waiting
  router::TopkSmem tk;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block too large");

template <int N>
DRB_DEV void bar_named(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(N) : "memory");
}

// Grid-wide barrier number `n` (1, 2, 3, ...): everyone adds one to a counter, then thread 0 of every block
// polls it until it reaches n * blocks. Measured on B200 (148 blocks): 1.3 us, the same as cooperative-groups
// grid.sync. A variant with one flag word per block, polled by a warp of every block, measured 3-7 us: any
// cache line that all 148 multiprocessors read at once is slow on this two-die L2, and fewer lines win.
// Bounded: ~2^17 polls, then the error word is set and `abort` makes every later barrier of this block fall
// through.
DRB_DEV void grid_barrier(Workspace* ws, Ctl& ctl, unsigned n) {
  __syncthreads();
  if (threadIdx.x == 0 && !ctl.abort) {
    __threadfence();
    atomicAdd(&ws->flags[0], 1u);
    const unsigned target = n * gridDim.x;
    bool ok = false;
    for (unsigned it = 0; it < (1u << 17); ++it) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&ws->flags[0]) : "memory");
      if (v >= target) {
        ok = true;
        break;
      }
      if (it > 256) __nanosleep(200);
      if (it > 1024 && *reinterpret_cast<volatile unsigned*>(&g_drb_error) != 0u) break;  // someone else gave up
    }
    if (!ok) {
      atomicMax(&g_drb_error, (unsigned)DRB_ERR_GRID_WAIT);
      ctl.abort = 1;
    }
  }
  __syncthreads();
}


__global__ void __launch_bounds__(THREADS, 1)
    k_moe_stack(const drb_moe_layer* __restrict__ layers, int n_layers, float* x, Workspace* ws, int E, float eps,
                int* __restrict__ idx_trace, float* __restrict__ wts_trace) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  float4* xs4 = reinterpret_cast<float4*>(dyn + CTL_BYTES);
  unsigned char* qx = dyn + CTL_BYTES + XS_BYTES;
  unsigned char* rw = qx + QX_BYTES;
  unsigned char* qa = rw + RW_BYTES;
  unsigned char* qs = qa + dn1::QA_BYTES;
  unsigned char* ring = qs + dn1::QS_BYTES;
  unsigned char* dst = ring + RING_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned G = gridDim.x, b = blockIdx.x;
  const gu1::Plan plan(b, G);
  const int n0 = (int)((long long)H * b / G), n1 = (int)((long long)H * (b + 1) / G), nr = n1 - n0;
  const int rrow0 = 2 * (int)b, nrr = max(0, min(2, E + 1 - rrow0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < gu1::STAGES; ++s) mbar_init(&ctl.gfull[s], 1);
    mbar_init(&ctl.dfull_routed, 1);
    mbar_init(&ctl.dfull_shared, 1);
    mbar_init(&ctl.rfull[0], 1);
    mbar_init(&ctl.rfull[1], 1);
    ctl.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // ---- producer-warp requests ------------------------------------------------------------------
  auto issue_router = [&](int l) {  // this block's two router rows of layer l
    if (lane == 0 && nrr > 0 && l < n_layers) {
      uint64_t* bar = &ctl.rfull[l & 1];
      mbar_expect_tx(bar, (unsigned)(nrr * H * 2));
      bulk_g2s(rw + (l & 1) * (2 * H * 2), static_cast<const unsigned char*>(layers[l].router) + (size_t)rrow0 * H * 2,
               (unsigned)(nrr * H * 2), bar);
    }
  };
  auto issue_shared_gu = [&](int l) {  // shared-expert gate/up chunks: lane t = chunk t
    if (l < n_layers && lane < plan.nsc) {
      bool shared;
      int base, ua, ub;
      plan.chunk(lane, shared, base, ua, ub);
      unsigned char* d = ring + (size_t)lane * gu1::STAGE_BYTES;
      const int n = ub - ua, slot = ua - base;
      const unsigned char* q = static_cast<const unsigned char*>(layers[l].sgu_q);
      const unsigned char* sp = static_cast<const unsigned char*>(layers[l].sgu_s);
      uint64_t* bar = &ctl.gfull[lane];
      mbar_expect_tx(bar, (unsigned)(n * 2 * (H + gu1::SSROW)));
      bulk_g2s(d + slot * H, q + (size_t)ua * H, (unsigned)(n * H), bar);
      bulk_g2s(d + (gu1::SU + slot) * H, q + ((size_t)I + ua) * H, (unsigned)(n * H), bar);
      bulk_g2s(d + 2 * gu1::SU * H + slot * gu1::SSROW, sp + (size_t)ua * gu1::SSROW, (unsigned)(n * gu1::SSROW), bar);
      bulk_g2s(d + 2 * gu1::SU * H + (gu1::SU + slot) * gu1::SSROW, sp + ((size_t)I + ua) * gu1::SSROW, (unsigned)(n * gu1::SSROW), bar);
    }
  };
  auto issue_shared_dn = [&](int l) {  // the shared expert's down rows of this block
    if (lane == 0 && l < n_layers && nr > 0) {
      mbar_expect_tx(&ctl.dfull_shared, (unsigned)(nr * I));
      bulk_g2s(dst + TOPK * dn::EXPERT_BYTES, static_cast<const unsigned char*>(layers[l].sd_q) + (size_t)n0 * I, (unsigned)(nr * I),
               &ctl.dfull_shared);
    }
  };
  auto issue_routed = [&](int l) {  // needs ctl.idx: lanes 0.. = routed gate/up chunks, lanes 16..23 = down rows per expert
    if (lane < plan.nrc) {
      const int t = plan.nsc + lane;
      bool shared;
      int base, ua, ub;
      plan.chunk(t, shared, base, ua, ub);
      unsigned char* d = ring + (size_t)t * gu1::STAGE_BYTES;
      const int n = ub - ua, slot = ua - base;
      const int k = ua / I, j = ua % I;
      const size_t ek = (size_t)ctl.idx[k];
      const unsigned char* q = static_cast<const unsigned char*>(layers[l].gu_q) + ek * (2 * I) * gu1::QROW;
      const unsigned char* smp = static_cast<const unsigned char*>(layers[l].gu_sm) + ek * (2 * I) * gu1::SMROW;
      uint64_t* bar = &ctl.gfull[t];
      mbar_expect_tx(bar, (unsigned)(n * 2 * (gu1::QROW + gu1::SMROW)));
      bulk_g2s(d + slot * gu1::QROW, q + (size_t)j * gu1::QROW, (unsigned)(n * gu1::QROW), bar);
      bulk_g2s(d + (gu1::RU + slot) * gu1::QROW, q + ((size_t)I + j) * gu1::QROW, (unsigned)(n * gu1::QROW), bar);
      bulk_g2s(d + 2 * gu1::RU * gu1::QROW + slot * gu1::SMROW, smp + (size_t)j * gu1::SMROW, (unsigned)(n * gu1::SMROW), bar);
      bulk_g2s(d + 2 * gu1::RU * gu1::QROW + (gu1::RU + slot) * gu1::SMROW, smp + ((size_t)I + j) * gu1::SMROW, (unsigned)(n * gu1::SMROW), bar);
    }
    if (nr > 0) {
      if (lane == 15) mbar_expect_tx(&ctl.dfull_routed, (unsigned)(nr * TOPK * (dn::QROW + dn::SMROW)));
      if (lane >= 16 && lane < 16 + TOPK) {
        const int k = lane - 16;
        const size_t row = (size_t)ctl.idx[k] * H + n0;
        bulk_g2s(dst + k * dn::EXPERT_BYTES, static_cast<const unsigned char*>(layers[l].d_q) + row * dn::QROW, (unsigned)(nr * dn::QROW),
                 &ctl.dfull_routed);
        bulk_g2s(dst + k * dn::EXPERT_BYTES + dn::RT * dn::QROW, static_cast<const unsigned char*>(layers[l].d_sm) + row * dn::SMROW,
                 (unsigned)(nr * dn::SMROW), &ctl.dfull_routed);
      }
    }
  };

  if (warp == CW) {
    issue_router(0);
    issue_shared_gu(0);
    issue_shared_dn(0);
  }
  unsigned nbar = 0;
  for (int l = 0; l < n_layers; ++l) {
    const drb_moe_layer L = layers[l];
    const unsigned par = l & 1;
    DRB_TRACE_POINT(0, 0);
    // ================= P0: normalise + quantise x, router logits =================
    if (warp < CW) {
      const float4 wv = reinterpret_cast<const float4*>(L.post_norm)[threadIdx.x];
      const float4 xv = __ldcg(reinterpret_cast<const float4*>(x) + threadIdx.x);
      const float ss = warp_sum(xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w);
      if (lane == 0) ctl.red[warp] = ss;
      bar_named<NT>(1);
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < CW; ++w) t += ctl.red[w];
      const float inv = rsqrtf(t / H + eps);
      const float4 xh = make_float4(xv.x * inv * wv.x, xv.y * inv * wv.y, xv.z * inv * wv.z, xv.w * inv * wv.w);
      xs4[threadIdx.x] = xh;
      quant_store_eo(qx, threadIdx.x, xh, true);
      bar_named<NT>(1);
      DRB_TRACE_POINT(1, 0);
      if (warp < 8 && nrr > 0) {  // threads 0..255: one 16-byte chunk (8 weights) of each of the block's two rows
        const float4 a = xs4[2 * threadIdx.x], c = xs4[2 * threadIdx.x + 1];
        unsigned long long xp[4] = {pack2(a.x, a.y), pack2(a.z, a.w), pack2(c.x, c.y), pack2(c.z, c.w)};
        mbar_wait(&ctl.rfull[par], (l >> 1) & 1, DRB_ERR_FULL_WAIT);
        const unsigned char* rows = rw + par * (2 * H * 2);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float d = 0.f;
          if (r < nrr) {
            float p0, p1;
            unpack2(dot8_bf16(*reinterpret_cast<const uint4*>(rows + (size_t)r * H * 2 + threadIdx.x * 16), xp, 0ull), p0, p1);
            d = p0 + p1;
          }
          d = warp_sum(d);
          if (lane == 0) ctl.rpart[r][warp] = d;
        }
        bar_named<256>(2);
        if ((int)threadIdx.x < nrr) {
          float tt = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) tt += ctl.rpart[threadIdx.x][w];
          __stcg(&ws->logits[rrow0 + threadIdx.x], tt);
        }
      }
    } else {
      issue_router(l + 1);
    }
    DRB_TRACE_POINT(2, 0);
    grid_barrier(ws, ctl, ++nbar);
    DRB_TRACE_POINT(3, 0);

    // ================= P1: every block derives the routing itself =================
    if (threadIdx.x < 256) {
      const int e = threadIdx.x;
      const float v = e < E ? __ldcg(&ws->logits[e]) : -INFINITY;
      if (v == 12345.678f) ctl.sgate = 0.f;  // keep the load before the probe
      DRB_TRACE_ANY(39, 0);
      router::softmax_topk<3>(v, E, TOPK, ctl.idx, ctl.wts, ctl.tk);
      if (e == 0) ctl.sgate = __ldcg(&ws->logits[E]);
    }
    __syncthreads();
    if (b == 0 && threadIdx.x < TOPK) {
      if (idx_trace) idx_trace[l * TOPK + threadIdx.x] = ctl.idx[threadIdx.x];
      if (wts_trace) wts_trace[l * TOPK + threadIdx.x] = ctl.wts[threadIdx.x];
    }
    DRB_TRACE_POINT(4, 0);
    if (warp == CW) issue_routed(l);

    // ================= P2: gate/up + SwiGLU on this block's share =================
    if (warp < CW) {
      QAct<32, true> x0, x1;
      float X0, X1;
      qact_load(x0, X0, qx + (size_t)lane * QB32_BYTES);
      qact_load(x1, X1, qx + (size_t)(32 + lane) * QB32_BYTES);
      const int nunits = plan.units();
      for (int o0 = warp; o0 < nunits; o0 += CW * 2) {
        float v[4];
        int uid[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int o = o0 + i * CW;
          v[2 * i] = v[2 * i + 1] = 0.f;
          uid[i] = -1;
          if (o >= nunits) continue;
          bool shared;
          int u, t, slot;
          plan.unit(o, shared, u, t, slot);
          uid[i] = shared ? TOPK * I + u : u;
          const unsigned char* st = ring + (size_t)t * gu1::STAGE_BYTES;
          mbar_wait(&ctl.gfull[t], par, DRB_ERR_FULL_WAIT);
          if (shared) {
            const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * H);
            const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(gu1::SU + slot) * H);
            const __half* gs = reinterpret_cast<const __half*>(st + 2 * gu1::SU * H + (size_t)slot * gu1::SSROW);
            const __half* us = reinterpret_cast<const __half*>(st + 2 * gu1::SU * H + (size_t)(gu1::SU + slot) * gu1::SSROW);
            v[2 * i] = __half2float(gs[lane >> 2]) * x0.delta * dot32_q8_eo(gr[2 * lane], gr[2 * lane + 1], x0, 0) +
                       __half2float(gs[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(gr[64 + 2 * lane], gr[64 + 2 * lane + 1], x1, 0);
            v[2 * i + 1] = __half2float(us[lane >> 2]) * x0.delta * dot32_q8_eo(ur[2 * lane], ur[2 * lane + 1], x0, 0) +
                           __half2float(us[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(ur[64 + 2 * lane], ur[64 + 2 * lane + 1], x1, 0);
          } else {
            const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)slot * gu1::QROW);
            const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(gu1::RU + slot) * gu1::QROW);
            const __half2* gs = reinterpret_cast<const __half2*>(st + 2 * gu1::RU * gu1::QROW + (size_t)slot * gu1::SMROW);
            const __half2* us = reinterpret_cast<const __half2*>(st + 2 * gu1::RU * gu1::QROW + (size_t)(gu1::RU + slot) * gu1::SMROW);
            const float2 g0 = __half22float2(gs[lane >> 1]), g1 = __half22float2(gs[16 + (lane >> 1)]);
            const float2 u0 = __half22float2(us[lane >> 1]), u1 = __half22float2(us[16 + (lane >> 1)]);
            v[2 * i] = g0.x * x0.delta * dot32_q4_i(gr[lane], x0, 0) + g0.y * X0 + g1.x * x1.delta * dot32_q4_i(gr[32 + lane], x1, 0) + g1.y * X1;
            v[2 * i + 1] = u0.x * x0.delta * dot32_q4_i(ur[lane], x0, 0) + u0.y * X0 + u1.x * x1.delta * dot32_q4_i(ur[32 + lane], x1, 0) + u1.y * X1;
          }
        }
        const bool hi16 = lane & 16, hi8 = lane & 8;
        const float r0 = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
        const float r1 = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
        float sres = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
        sres += __shfl_xor_sync(0xffffffffu, sres, 4);
        sres += __shfl_xor_sync(0xffffffffu, sres, 2);
        sres += __shfl_xor_sync(0xffffffffu, sres, 1);
        const float upv = __shfl_xor_sync(0xffffffffu, sres, 8);
        if ((lane & 15) == 0) {
          const int id = (lane & 16) ? uid[1] : uid[0];
          if (id >= 0) __stcg(&ws->act[id], silu_f(sres) * upv);
        }
      }
    }
    DRB_TRACE_POINT(5, 0);
    grid_barrier(ws, ctl, ++nbar);
    DRB_TRACE_POINT(6, 0);
    if (warp == CW) issue_shared_gu(l + 1);  // the ring is free again

    // ================= P3: down + combine on this block's rows =================
    if (warp < CW) {
      const int ke = warp & (TOPK - 1), rh = warp >> 3;
      const float ssc = warp < nr ? __half2float(__ldg(static_cast<const __half*>(L.sd_s) + (size_t)(n0 + warp) * (I / 128) + (lane >> 3))) : 0.f;
      const float xres = (int)threadIdx.x < nr ? __ldcg(x + n0 + threadIdx.x) : 0.f;  // residual, fetched early
      const float sgv = sigmoid_f(ctl.sgate);
      constexpr int NR4 = TOPK * I / 4, NS4 = I / 4;
      constexpr int AV = (NR4 + NS4 + NT - 1) / NT;
      float4 av[AV];
#pragma unroll
      for (int i = 0; i < AV; ++i) {
        const int g = threadIdx.x + i * NT;
        av[i] = g < NR4 + NS4 ? __ldcg(reinterpret_cast<const float4*>(ws->act) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < AV; ++i) {
        const int g = threadIdx.x + i * NT;
        if (g - lane < NR4) quant_store_eo(qa, g, av[i], true);
        else quant_store_nat(qs, g - NR4, av[i], g < NR4 + NS4);
      }
      bar_named<NT>(1);
      DRB_TRACE_POINT(7, 0);
      const int cc = lane & 15, half = lane >> 4;
      QAct<32, true> aq;
      float A;
      qact_load(aq, A, qa + (size_t)(ke * (I / 32) + cc) * QB32_BYTES);
      QAct<16, false> sq;
      qact_load(sq, qs + (size_t)lane * QB16_BYTES);
      if (nr > 0) {
        mbar_wait(&ctl.dfull_routed, par, DRB_ERR_FULL_WAIT);
        mbar_wait(&ctl.dfull_shared, par, DRB_ERR_FULL_WAIT);
      }
      const unsigned char* eq = dst + ke * dn::EXPERT_BYTES;
      const unsigned char* esm = eq + dn::RT * dn::QROW;
      float v[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int lr = 2 * (rh * 4 + p) + half;
        v[p] = 0.f;
        if (lr < nr) {
          const uint4 w = *reinterpret_cast<const uint4*>(eq + (size_t)lr * dn::QROW + 16 * cc);
          const float2 sm = __half22float2(*reinterpret_cast<const __half2*>(esm + (size_t)lr * dn::SMROW + 4 * (cc >> 1)));
          v[p] = sm.x * aq.delta * dot32_q4_i(w, aq, 0) + sm.y * A;
        }
      }
      {
        const bool hi8 = lane & 8, hi4 = lane & 4;
        const float r0 = (hi8 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi8 ? v[0] : v[2], 8);
        const float r1 = (hi8 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi8 ? v[1] : v[3], 8);
        float sres = (hi4 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi4 ? r0 : r1, 4);
        sres += __shfl_xor_sync(0xffffffffu, sres, 2);
        sres += __shfl_xor_sync(0xffffffffu, sres, 1);
        const int p = (hi8 ? 2 : 0) + (hi4 ? 1 : 0);
        const int lr = 2 * (rh * 4 + p) + half;
        if ((lane & 3) == 0 && lr < nr) ctl.part[ke][lr] = sres;
      }
      {
        float sres = 0.f;
        if (warp < nr) sres = ssc * sq.delta * dot16_q8_i(*reinterpret_cast<const uint4*>(dst + TOPK * dn::EXPERT_BYTES + (size_t)warp * I + 16 * lane), sq, 0);
        sres = warp_sum(sres);
        if (lane == 0 && warp < nr) ctl.part[TOPK][warp] = sres;
      }
      bar_named<NT>(1);
      if ((int)threadIdx.x < nr) {
        const int lr = threadIdx.x;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < TOPK; ++k) acc += ctl.wts[k] * ctl.part[k][lr];
        x[n0 + lr] = xres + sgv * ctl.part[TOPK][lr] + acc;
      }
    }
    DRB_TRACE_POINT(8, 0);
    grid_barrier(ws, ctl, ++nbar);
    DRB_TRACE_POINT(9, 0);
    if (warp == CW) issue_shared_dn(l + 1);  // the down stage is free again
  }
}

static cudaError_t configure_all() {
  cudaError_t e = cudaFuncSetAttribute(k_moe_stack, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return drb_carveout(k_moe_stack);
}
}  // namespace stack

// Bytes of device workspace drb_moe_stack_decode needs (any contents; the call zeroes what it must).
extern "C" int drb_moe_stack_workspace_bytes(void) { return (int)sizeof(stack::Workspace); }

// x <- x + moe_l(rmsnorm(x)) for l = 0 .. n_layers - 1, in place, in one cooperative kernel launch.
// layers: device array of n_layers drb_moe_layer. workspace: drb_moe_stack_workspace_bytes() bytes of
// device memory, 256-byte aligned. idx_trace / wts_trace: optional device arrays [n_layers, topk]
// receiving every layer's routing (NULL to skip). Only h = 2048, i = 512, topk = 8, e <= 256, and a
// device with at least 148 multiprocessors are supported (-1 otherwise). Capturable in a graph.
// Calls that share a workspace must not overlap on the GPU.
extern "C" int drb_moe_stack_decode(const drb_moe_layer* layers, int n_layers, float* x, void* workspace, int e, int topk,
                                    int h, int i, float eps, int* idx_trace, float* wts_trace, cudaStream_t st) {
  if (h != moe::H || i != moe::I || topk != moe::TOPK || e < topk || e > stack::MAX_E || n_layers < 0) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (dev.sms < stack::gu1::MIN_GRID) return -1;
  if (n_layers == 0) return 0;
  stack::Workspace* ws = static_cast<stack::Workspace*>(workspace);
  if (dev.sms > stack::MAX_BLOCKS) return -1;
  cudaError_t err = cudaMemsetAsync(ws->flags, 0, sizeof(ws->flags), st);
  if (err != cudaSuccess) return (int)err;
  void* args[] = {(void*)&layers, (void*)&n_layers, (void*)&x, (void*)&ws, (void*)&e, (void*)&eps, (void*)&idx_trace, (void*)&wts_trace};
  err = cudaLaunchCooperativeKernel((const void*)stack::k_moe_stack, dim3(dev.sms), dim3(stack::THREADS), args, stack::SMEM_BYTES, st);
  return err == cudaSuccess ? 0 : (int)err;
}
