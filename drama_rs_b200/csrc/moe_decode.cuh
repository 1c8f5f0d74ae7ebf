// Batch-1 MoE decode: dr_moe_decode = gate/up + SwiGLU over the 8 routed int4 experts and the int8
// shared expert, then down projection + weighted combine + sigmoid-gated shared expert + residual.
//
// Gate/up: 144 blocks. Block b < 128 owns 32 consecutive units (a gate row and its up row each) of one routed
// expert, blocks 128..143 own 32 units of the shared expert; every block requests ALL its rows at once with bulk
// asynchronous copies (four parts, one mbarrier each), so the HBM queue is full from the first microsecond, and the
// shared expert's rows, which do not depend on the routing, are requested before the dependency wait. The 32
// activations a block produces are exactly one quantisation block of the down projection's input, so the block
// converts them to block fixed point itself and the down kernel never sees floats.
// Down: at least 128 blocks of at most 16 output rows; a block pulls its rows of the eight chosen experts and of the
// shared expert into shared memory before it waits for the activations (programmatic dependent launch), copies the
// 16 KB of quantised activations once, and its lanes keep the limb words of their k-slice in registers.
//
// x is read coalesced, normalised, and converted once per block to block fixed point (three signed 7-bit limbs per
// value, see common.cuh). Weight words then go through dp4a against the limbs: integer-exact sums, group scales
// applied in fp32, warp-shuffle reductions folded over all the rows a warp owns.
//
// Every load of data that the preceding kernel wrote goes through ld.global.cg (or a bulk copy): a block launched
// programmatically can be resident before its predecessor has written that data, and an L1-cached or non-coherent
// load may then return what the multiprocessor saw earlier. Measured: with plain loads a 3-layer stack diverged.
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

// The SwiGLU activations cross from gate/up to down as block fixed point, not as floats: `act` (the caller's
// scratch of (topk + 1) * I floats, which nothing else reads) holds, for every 32 consecutive inputs of a routed
// expert's down projection, one 112-byte block (limbs in even/odd order, delta, sum; common.cuh), block
// k * 16 + c for inputs [32 c, 32 c + 32) of expert slot k; then, from ACTQ_SHARED on, one 64-byte block (natural
// order) for every 16 inputs of the shared expert. 16,384 of the 18,432 bytes are used. Every gate/up block
// produces exactly the 32 values of one routed block (or two shared ones), so it quantises them once and the down
// kernel's lanes load their limbs straight into registers.
constexpr int ACTQ_SHARED = TOPK * (I / 32) * QB32_BYTES;  // 14,336

namespace gu {

constexpr int CW = 16;                                    // consumer warps
constexpr int NT = CW * 32;                               // consumer threads
constexpr int THREADS = NT + 32;                          // + one producer warp
constexpr int UNITS = 32;                                 // units (gate row + up row) per block: warp w takes w and w + 16
constexpr int ROUTED_BLOCKS = TOPK * I / UNITS;           // 128
constexpr int SHARED_BLOCKS = I / UNITS;                  // 16
constexpr int GRID = ROUTED_BLOCKS + SHARED_BLOCKS;       // 144
constexpr int QUARTERS = 4, QU = UNITS / QUARTERS;  // the block's rows arrive in parts of QU units, one mbarrier each
constexpr int QROW = H / 2;                               // 1024 bytes of nibbles per routed row
constexpr int SMROW = (H / 64) * 4;                       // 128 bytes of (scale, min) per routed row
constexpr int SSROW = (H / 128) * 2;                      // 32 bytes of scales per shared-expert row
// stage: gate rows [32] | up rows [32] | gate scales [32] | up scales [32]
constexpr int R_STAGE = 2 * UNITS * (QROW + SMROW);       // 73,728
constexpr int S_STAGE = 2 * UNITS * (H + SSROW);          // 133,120
constexpr int CTL_BYTES = 1024;
constexpr int QX_BYTES = (H / 32) * QB32_BYTES;           // the normalised activations as limb blocks
constexpr size_t SMEM_BYTES = CTL_BYTES + QX_BYTES + (size_t)S_STAGE;
static_assert(NT == H / 4, "one float4 of x per consumer thread");

struct Ctl {
  uint64_t full[QUARTERS];
  float red[CW];
  float actv[UNITS];
};

// One warp turns 32 values (lane = input index) into a 112-byte even/odd block at dst (global or shared).
DRB_DEV void quant_block32_warp(float v, unsigned char* dst, int lane) {
  const float m = warp_max(fabsf(v));
  const float sum = warp_sum(v);
  const float delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
  int l0, l1, l2;
  limbs3(__float2int_rn(v * (1.f / delta)), l0, l1, l2);
  const uint32_t pack = (uint32_t)(l0 & 0xff) | ((uint32_t)(l1 & 0xff) << 8) | ((uint32_t)(l2 & 0xff) << 16);
  // word w (lanes 0..7) holds inputs 8 (w / 2) + (w & 1) + {0, 2, 4, 6}
  const int base = 8 * ((lane >> 1) & 3) + (lane & 1);
  const uint32_t t0 = __shfl_sync(0xffffffffu, pack, base), t1 = __shfl_sync(0xffffffffu, pack, base + 2);
  const uint32_t t2 = __shfl_sync(0xffffffffu, pack, base + 4), t3 = __shfl_sync(0xffffffffu, pack, base + 6);
  if (lane < 8) {
    uint32_t* out = reinterpret_cast<uint32_t*>(dst);
    out[lane] = prmt(prmt(t0, t1, 0x0040u), prmt(t2, t3, 0x0040u), 0x5410u);
    out[8 + lane] = prmt(prmt(t0, t1, 0x0051u), prmt(t2, t3, 0x0051u), 0x5410u);
    out[16 + lane] = prmt(prmt(t0, t1, 0x0062u), prmt(t2, t3, 0x0062u), 0x5410u);
  }
  if (lane == 0) {
    *reinterpret_cast<float*>(dst + 96) = delta;
    *reinterpret_cast<float*>(dst + 100) = sum;
  }
}

// Each half-warp turns 16 values (lane & 15 = input index) into a 64-byte natural-order block at dst + 64 * half.
DRB_DEV void quant_block16_halfwarps(float v, unsigned char* dst, int lane) {
  float m = fabsf(v);
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
  int l0, l1, l2;
  limbs3(__float2int_rn(v * (1.f / delta)), l0, l1, l2);
  const uint32_t pack = (uint32_t)(l0 & 0xff) | ((uint32_t)(l1 & 0xff) << 8) | ((uint32_t)(l2 & 0xff) << 16);
  const int h = lane >> 4, q = lane & 3;  // word q (lanes 0..3 of the half) holds inputs 4 q .. 4 q + 3
  const int base = 16 * h + 4 * q;
  const uint32_t t0 = __shfl_sync(0xffffffffu, pack, base), t1 = __shfl_sync(0xffffffffu, pack, base + 1);
  const uint32_t t2 = __shfl_sync(0xffffffffu, pack, base + 2), t3 = __shfl_sync(0xffffffffu, pack, base + 3);
  unsigned char* blk = dst + h * QB16_BYTES;
  if ((lane & 15) < 4) {
    uint32_t* out = reinterpret_cast<uint32_t*>(blk);
    out[q] = prmt(prmt(t0, t1, 0x0040u), prmt(t2, t3, 0x0040u), 0x5410u);
    out[4 + q] = prmt(prmt(t0, t1, 0x0051u), prmt(t2, t3, 0x0051u), 0x5410u);
    out[8 + q] = prmt(prmt(t0, t1, 0x0062u), prmt(t2, t3, 0x0062u), 0x5410u);
  }
  if ((lane & 15) == 0) *reinterpret_cast<float*>(blk + 48) = delta;
}

// Block b < 128: units [32 (b % 16), +32) of routed expert slot b / 16 (64 int4 rows, 72 KB). Block b >= 128: units
// [32 (b - 128), +32) of the shared expert (64 int8 rows, 130 KB; they do not depend on the routing and are requested
// before the dependency wait, so these larger blocks finish first). The rows arrive in four parts of 8 units with one
// mbarrier each; warp w computes units w and w + 16, i.e. parts w / 8 and 2 + w / 8.
__global__ void __launch_bounds__(THREADS, 1)
    k_moe_gate_up(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
                  const __half* __restrict__ shs, const float* __restrict__ x, const int* __restrict__ idx,
                  unsigned char* __restrict__ actq, const float* __restrict__ nw, float eps) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* qx = dyn + CTL_BYTES;
  unsigned char* st = dyn + CTL_BYTES + QX_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x;
  const bool shared = b >= ROUTED_BLOCKS;
  const int j0 = shared ? (b - ROUTED_BLOCKS) * UNITS : (b % (I / UNITS)) * UNITS;  // first unit

  if (threadIdx.x == 0) {
    for (int q = 0; q < QUARTERS; ++q) mbar_init(&ctl.full[q], 1);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // ---------------- producer warp: lane 4 q + c requests copy c (gate rows, up rows, gate scales, up scales) of part q
    const int q = lane >> 2, c = lane & 3;
    const bool issuing = q < QUARTERS;
    if (shared) {
      if (issuing && c == 0) mbar_expect_tx(&ctl.full[q], (unsigned)(2 * QU * (H + SSROW)));
      __syncwarp();
      if (issuing) {
        const int u0 = j0 + q * QU, l0 = q * QU;
        const unsigned char* sp = reinterpret_cast<const unsigned char*>(shs);
        if (c == 0) bulk_g2s(st + (size_t)l0 * H, shq + (size_t)u0 * H, QU * H, &ctl.full[q]);
        else if (c == 1) bulk_g2s(st + (size_t)(UNITS + l0) * H, shq + ((size_t)I + u0) * H, QU * H, &ctl.full[q]);
        else if (c == 2) bulk_g2s(st + (size_t)2 * UNITS * H + l0 * SSROW, sp + (size_t)u0 * SSROW, QU * SSROW, &ctl.full[q]);
        else bulk_g2s(st + (size_t)2 * UNITS * H + (UNITS + l0) * SSROW, sp + ((size_t)I + u0) * SSROW, QU * SSROW, &ctl.full[q]);
      }
      pdl_wait();
    } else {
      pdl_wait();  // idx is the router's output
      if (issuing && c == 0) mbar_expect_tx(&ctl.full[q], (unsigned)(2 * QU * (QROW + SMROW)));
      __syncwarp();
      if (issuing) {
        const size_t ek = (size_t)__ldcg(idx + b / (I / UNITS));
        const uint8_t* qp = Q + ek * (2 * I) * QROW;
        const unsigned char* smp = reinterpret_cast<const unsigned char*>(SM) + ek * (2 * I) * SMROW;
        const int u0 = j0 + q * QU, l0 = q * QU;
        if (c == 0) bulk_g2s(st + (size_t)l0 * QROW, qp + (size_t)u0 * QROW, QU * QROW, &ctl.full[q]);
        else if (c == 1) bulk_g2s(st + (size_t)(UNITS + l0) * QROW, qp + ((size_t)I + u0) * QROW, QU * QROW, &ctl.full[q]);
        else if (c == 2) bulk_g2s(st + (size_t)2 * UNITS * QROW + l0 * SMROW, smp + (size_t)u0 * SMROW, QU * SMROW, &ctl.full[q]);
        else bulk_g2s(st + (size_t)2 * UNITS * QROW + (UNITS + l0) * SMROW, smp + ((size_t)I + u0) * SMROW, QU * SMROW, &ctl.full[q]);
      }
    }
    pdl_launch_dependents();  // never before the wait: the down kernel's prologue reads the router's idx
    return;
  }

  // ---------------- consumers
  // The norm weight is a constant: fetch it before the dependency wait. Thread t owns float4 t.
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
  quant_store_eo(qx, threadIdx.x, make_float4(xv.x * inv * wv.x, xv.y * inv * wv.y, xv.z * inv * wv.z, xv.w * inv * wv.w), true);
  named_sync<NT>();
  // This lane owns k in [32 lane, +32) and [1024 + 32 lane, +32): 16-byte chunks lane and 32 + lane of an int4
  // row, chunks {2 lane, 2 lane + 1} and {64 + 2 lane, 64 + 2 lane + 1} of an int8 row.
  QAct<32, true> x0, x1;
  float X0, X1;
  qact_load(x0, X0, qx + (size_t)lane * QB32_BYTES);
  qact_load(x1, X1, qx + (size_t)(32 + lane) * QB32_BYTES);

  // v[2i] = gate, v[2i + 1] = up partial sums of this warp's unit warp + 16 i
  float v[4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int u = warp + CW * i;
    mbar_wait(&ctl.full[u / QU], 0, DRB_ERR_FULL_WAIT);
    if (shared) {
      const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)u * H);
      const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(UNITS + u) * H);
      const __half* gs = reinterpret_cast<const __half*>(st + (size_t)2 * UNITS * H + (size_t)u * SSROW);
      const __half* us = reinterpret_cast<const __half*>(st + (size_t)2 * UNITS * H + (size_t)(UNITS + u) * SSROW);
      v[2 * i] = __half2float(gs[lane >> 2]) * x0.delta * dot32_q8_eo(gr[2 * lane], gr[2 * lane + 1], x0, 0) +
                 __half2float(gs[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(gr[64 + 2 * lane], gr[64 + 2 * lane + 1], x1, 0);
      v[2 * i + 1] = __half2float(us[lane >> 2]) * x0.delta * dot32_q8_eo(ur[2 * lane], ur[2 * lane + 1], x0, 0) +
                     __half2float(us[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(ur[64 + 2 * lane], ur[64 + 2 * lane + 1], x1, 0);
    } else {
      const uint4* gr = reinterpret_cast<const uint4*>(st + (size_t)u * QROW);
      const uint4* ur = reinterpret_cast<const uint4*>(st + (size_t)(UNITS + u) * QROW);
      const __half2* gs = reinterpret_cast<const __half2*>(st + (size_t)2 * UNITS * QROW + (size_t)u * SMROW);
      const __half2* us = reinterpret_cast<const __half2*>(st + (size_t)2 * UNITS * QROW + (size_t)(UNITS + u) * SMROW);
      // w = s*q + m: sum_k w x = s * delta * sum(q n) + m * sum(x) per 64-group; chunk c belongs to group c / 2.
      const float2 g0 = __half22float2(gs[lane >> 1]), g1 = __half22float2(gs[16 + (lane >> 1)]);
      const float2 u0 = __half22float2(us[lane >> 1]), u1 = __half22float2(us[16 + (lane >> 1)]);
      v[2 * i] = g0.x * x0.delta * dot32_q4_i(gr[lane], x0, 0) + g0.y * X0 + g1.x * x1.delta * dot32_q4_i(gr[32 + lane], x1, 0) + g1.y * X1;
      v[2 * i + 1] = u0.x * x0.delta * dot32_q4_i(ur[lane], x0, 0) + u0.y * X0 + u1.x * x1.delta * dot32_q4_i(ur[32 + lane], x1, 0) + u1.y * X1;
    }
  }
  // Fold the four per-lane sums into one reduction: after two exchange steps lane group
  // (lane & 16, lane & 8) carries v[(lane >> 3) & 3]; three butterfly steps finish it.
  const bool hi16 = lane & 16, hi8 = lane & 8;
  const float r0 = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
  const float r1 = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
  float s = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  // lanes 0..7: gate of unit warp, 8..15: its up, 16..23: gate of unit warp + 16, 24..31: its up
  const float upv = __shfl_xor_sync(0xffffffffu, s, 8);
  if ((lane & 15) == 0) ctl.actv[warp + (lane & 16)] = silu_f(s) * upv;
  named_sync<NT>();
  if (warp == 0) {
    const float a = ctl.actv[lane];
    if (shared) quant_block16_halfwarps(a, actq + ACTQ_SHARED + (size_t)(b - ROUTED_BLOCKS) * 2 * QB16_BYTES, lane);
    else quant_block32_warp(a, actq + (size_t)b * QB32_BYTES, lane);
  }
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
constexpr int ACTQ_BYTES = TOPK * (I / 32) * QB32_BYTES + (I / 16) * QB16_BYTES;  // 16,384: the gate/up kernel's output
constexpr size_t SMEM_BYTES = CTL_BYTES + ACTQ_BYTES + STAGE_BYTES;
static_assert(ACTQ_BYTES == 2 * NT * 16, "two 16-byte pieces of the activations per consumer thread");
static_assert(RT == CW, "one shared-expert row per consumer warp");

struct Ctl {
  uint64_t full;
  float part[TOPK + 1][RT];
  float wk[TOPK]; // the routing weights and the shared expert's gate, fetched once per block
  float sgate;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block too large");

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_down(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const int8_t* __restrict__ shq,
               const __half* __restrict__ shs, const unsigned char* __restrict__ actq, const int* __restrict__ idx,
               const float* __restrict__ wts, const float* __restrict__ sgate, const float* res, float* y,
               const char* pf, size_t pf_bytes) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* qa = dyn + CTL_BYTES;
  unsigned char* st = qa + ACTQ_BYTES;
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
    // ---------------- producer warp. This kernel is only ever launched behind k_moe_gate_up, which lets its
    // dependents start after its own dependency wait: the routing is final by the time we get here.
    // Lane k < 8 requests expert slot k's rows, lane 8 the shared expert's.
    if (nr > 0) {
      if (lane == 0) mbar_expect_tx(&ctl.full, (unsigned)(nr * (TOPK * (QROW + SMROW) + I)));
      __syncwarp();
      if (lane < TOPK) {
        const size_t row = (size_t)__ldcg(idx + lane) * H + n0;
        bulk_g2s(st + lane * EXPERT_BYTES, Q + row * QROW, (unsigned)(nr * QROW), &ctl.full);
        bulk_g2s(st + lane * EXPERT_BYTES + RT * QROW, reinterpret_cast<const unsigned char*>(SM) + row * SMROW,
                 (unsigned)(nr * SMROW), &ctl.full);
      } else if (lane == TOPK) {
        bulk_g2s(st + TOPK * EXPERT_BYTES, shq + (size_t)n0 * I, (unsigned)(nr * I), &ctl.full);
      }
    }
    if (lane == 0) prefetch_share(pf, pf_bytes, b, G);
    return;
  }

  // ---------------- consumers
  const int ke = warp & (TOPK - 1), rh = warp >> 3;
  // The shared expert's scales are constants: fetched before the dependency wait.
  const float ssc = warp < nr ? __half2float(__ldg(shs + (size_t)(n0 + warp) * (I / 128) + (lane >> 3))) : 0.f;
  pdl_wait();  // the activations, and everything the caller wrote before
  // The block copies the 16 KB of activations once (read at L2: they were written while this block may already
  // have been resident, so nothing of them may come from this multiprocessor's L1), together with the routing
  // weights; then half-warps take alternate rows, lane & 15 = 16-byte chunk cc of the row, k in [32 cc, 32 cc + 32):
  // its activations are block ke * 16 + cc.
  {
    const uint4* src = reinterpret_cast<const uint4*>(actq);
    const uint4 p0 = __ldcg(src + threadIdx.x), p1 = __ldcg(src + NT + threadIdx.x);
    float r = 0.f;
    if (threadIdx.x < TOPK) r = __ldcg(wts + threadIdx.x);
    else if (threadIdx.x == TOPK) r = __ldcg(sgate);
    reinterpret_cast<uint4*>(qa)[threadIdx.x] = p0;
    reinterpret_cast<uint4*>(qa)[NT + threadIdx.x] = p1;
    if (threadIdx.x < TOPK) ctl.wk[threadIdx.x] = r;
    else if (threadIdx.x == TOPK) ctl.sgate = r;
  }
  named_sync<NT>();
  const int cc = lane & 15, half = lane >> 4;
  QAct<32, true> aq;
  float A;
  qact_load(aq, A, qa + (size_t)(ke * (I / 32) + cc) * QB32_BYTES);
  QAct<16, false> sq;  // shared expert: the whole warp per row, lane = 16-byte chunk of 16 int8
  qact_load(sq, qa + ACTQ_SHARED + (size_t)lane * QB16_BYTES);
  const float sg = sigmoid_f(ctl.sgate);
  float wk[TOPK];
#pragma unroll
  for (int k = 0; k < TOPK; ++k) wk[k] = ctl.wk[k];

  mbar_wait(&ctl.full, 0, DRB_ERR_FULL_WAIT);
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
    const float yn = __ldcg(res + n0 + lr) + sg * ctl.part[TOPK][lr] + acc;
    y[n0 + lr] = yn;
  }
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

// act must hold (topk + 1) * I floats; between the two kernels it carries the activations as block fixed point
// (see ACTQ_SHARED above), not as floats. x, res and y may be one buffer (the reference's caller passes the
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
  const int g_gu = moe::gu::GRID;
  const int g_dn = dev.sms > moe::dn::MIN_GRID ? dev.sms : moe::dn::MIN_GRID;
  drb_launch(moe::gu::k_moe_gate_up, dim3(g_gu), dim3(moe::gu::THREADS), moe::gu::SMEM_BYTES, st, dev.pdl, gu_q, gu_sm,
             sgu_q, sgu_s, x, idx, reinterpret_cast<unsigned char*>(act), nw, eps);
  drb_launch(moe::dn::k_moe_down, dim3(g_dn), dim3(moe::dn::THREADS), moe::dn::SMEM_BYTES, st, dev.pdl, d_q, d_sm, sd_q,
             sd_s, reinterpret_cast<const unsigned char*>(act), idx, wts, sgate, res, y, pf, pf_bytes);
  return 0;
}
