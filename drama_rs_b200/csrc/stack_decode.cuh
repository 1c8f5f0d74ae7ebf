// drb_moe_stack_decode: a whole stack of MoE layers at batch 1 in ONE persistent kernel.
//
//   for each layer:  x <- x + moe_l(rmsnorm(x, post_norm_l))
//
// This is the 40-layer decode step of the benchmark (hidden state carried layer to layer). It has no
// counterpart in the reference's ABI (there the token mixer sits between two MoE blocks); the per-layer
// entry points dr_router_topk and dr_moe_decode remain the drop-in path and compute the same thing.
//
// One block per multiprocessor, launched cooperatively (all blocks resident). A batch-1 layer is a chain
// of three all-to-all hand-overs (logits -> routing, activations -> down projection, hidden state -> next
// layer) around 18 MB of weight streaming, so what decides its duration is the cost of a hand-over, not
// bandwidth. Nothing here uses a grid-wide barrier. Every value that crosses blocks travels as a 64-bit
// word {payload, tag} written with one store and polled with plain loads by whoever needs it: the tag is
// the layer number, a word is valid when its tag matches, and an aligned 64-bit access cannot tear. A
// hand-over then costs one store and one load through L2 instead of store + fence + flag + poll + load,
// and a consumer starts on the first words that arrive instead of waiting for the slowest producer.
//
//   hidden state   y[2048]        {f32, tag}; written by the block that owns the row, read by every block
//   router logits  logits[E + 1]  {f32, tag}; block b computes rows 2b, 2b + 1
//   activations    routed: per 32 inputs of the down projection 24 limb words + delta + sum (the
//                  block-fixed-point form of common.cuh), shared expert: per 16 inputs 12 limb words + delta;
//                  one {word, tag} each, written by the gate/up block that produced the 32 values
//
// Work split per layer (G >= 144 blocks):
//   gate/up  block b < 128: 32 units (gate row + up row) of routed expert slot b / 16; blocks 128..143: 32 units
//            of the shared expert. All of a block's rows are requested at once (bulk copies, four mbarriers).
//   down     block b: rows [2048 b / G, 2048 (b + 1) / G) of all eight chosen experts and of the shared expert.
//   router   block b: rows 2b, 2b + 1 of the [E + 1, 2048] matrix; the eight warps of every block then derive the
//            top-8 themselves from the E + 1 logits (identical everywhere), so the routing needs no second hand-over.
// The producer warp requests the routed rows (gate/up and down) the moment the routing is known; rows that do
// not depend on the routing (router, shared expert) are requested as soon as their buffer is free, up to a
// layer ahead.
//
// Every wait is bounded: a poll that runs out sets the device error word and the block's abort flag, after
// which no wait of that block spins again and the kernel runs to its end.
#pragma once

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

constexpr int CW = 16;             // consumer warps
constexpr int NT = CW * 32;        // consumer threads
constexpr int THREADS = NT + 32;   // + the producer warp
constexpr int MAX_E = 256;

// gate/up
constexpr int UNITS = 32;                       // units per block; warp w takes units w and w + 16
constexpr int ROUTED_UB = TOPK * I / UNITS;     // 128 blocks of routed units
constexpr int SHARED_UB = I / UNITS;            // 16 blocks of shared-expert units
constexpr int UNIT_BLOCKS = ROUTED_UB + SHARED_UB;
constexpr int MIN_GRID = UNIT_BLOCKS;           // also >= (MAX_E + 2) / 2 router-row pairs and <= 16 down rows per block
constexpr int MAX_GRID = 1024;
constexpr int PARTS = 4, PU = UNITS / PARTS;    // a block's rows arrive in four parts of eight units
constexpr int QROW = H / 2;                     // bytes of nibbles per routed gate/up row
constexpr int SMROW = (H / 64) * 4;             // bytes of (scale, min) per routed gate/up row
constexpr int SSROW = (H / 128) * 2;            // bytes of scales per shared-expert gate/up row
constexpr int GU_STAGE_R = 2 * UNITS * (QROW + SMROW);  // 73,728
constexpr int GU_STAGE_S = 2 * UNITS * (H + SSROW);     // 133,120

// down
constexpr int RT = 16;                          // rows per block at most
constexpr int DQROW = I / 2;                    // 256 bytes of nibbles per routed down row
constexpr int DSMROW = (I / 64) * 4;            // 32 bytes of (scale, min)
constexpr int D_EXPERT = RT * (DQROW + DSMROW);
constexpr int D_STAGE = TOPK * D_EXPERT + RT * I;  // 45,056

// hand-over buffers
constexpr int ACT_R_WORDS = 26;  // per routed block of 32 inputs: limbs [3][8] (even/odd order), delta, sum
constexpr int ACT_S_WORDS = 14;  // per shared block of 16 inputs: limbs [3][4] (natural order), delta, pad
// Everything that crosses blocks, as tagged words. The kernel can keep `reps` replicas of it (producers write all
// of them, block b reads replica b % reps) so that fewer blocks poll the same cache lines; measured, more than one
// replica buys nothing (the polls are whole-line requests that L2 serves in a few hundred nanoseconds whatever
// their number), so every launch passes reps = 1. The count stays a run-time value all the same: with it folded
// into the code the same kernel measured 11.45 us per layer instead of 10.85, a matter of the compiler's schedule
// around the tagged stores and polls.
struct alignas(128) Copy {
  unsigned long long y[H];
  unsigned long long logits[MAX_E + 8];
  unsigned long long act_r[ROUTED_UB * ACT_R_WORDS];
  unsigned long long act_s[2 * SHARED_UB * ACT_S_WORDS];
};
constexpr int COPY_WORDS = (int)(sizeof(Copy) / sizeof(unsigned long long));
static_assert(sizeof(Copy) % 128 == 0 && (sizeof(unsigned long long) * (H + MAX_E + 8)) % 16 == 0, "aligned sections");

// shared memory map
constexpr int CTL_BYTES = 4096;
constexpr int QX_BYTES = (H / 32) * QB32_BYTES;       // normalised x as limb blocks (gate/up)
constexpr int RW_BYTES = 2 * H * 2;                   // this block's two router rows
constexpr int QS_BYTES = (I / 16) * QB16_BYTES;       // the shared expert's activations as limb blocks (down)
constexpr int PA_WARP_BYTES = 8 * ACT_R_WORDS * 4;     // a warp's eight routed activation blocks, payload words only
constexpr int PA_BYTES = CW * PA_WARP_BYTES;
constexpr size_t SMEM_BYTES = CTL_BYTES + QX_BYTES + RW_BYTES + QS_BYTES + PA_BYTES + GU_STAGE_S + D_STAGE;
static_assert(SMEM_BYTES <= 232448, "does not fit one multiprocessor");

// named barriers (0 is __syncthreads)
constexpr int BAR_CONS = 1;   // the 512 consumer threads
constexpr int BAR_TOPK = 2;   // warps 0..7 inside softmax_topk
constexpr int BAR_IDX = 3;    // warps 0..7 arrive, the producer waits: the routing is in shared memory
constexpr int BAR_GU = 4;     // consumers arrive, the producer waits: the gate/up stage is free
constexpr int BAR_DN = 5;     // consumers arrive, the producer waits: the down stage is free
constexpr int BAR_RT = 6;     // warps 0, 1 arrive, the producer waits: the router rows are free

struct Ctl {
  uint64_t gfull[PARTS];
  uint64_t dfull_r, dfull_s, rfull;
  float red[3][CW];  // per warp: sum of squares, the two router rows' partial dot products
  float actv[UNITS];
  float part[TOPK][2][RT];
  float part_s[RT];
  int idx[TOPK];
  float wts[TOPK];
  float sgate;
  int abort;  // a wait of this block ran out: no wait spins again
  router::TopkSmem tk;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block too large");

template <int N>
DRB_DEV void bar_sync(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(N) : "memory");
}
template <int N>
DRB_DEV void bar_arrive(int id) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(N) : "memory");
}

// ---- tagged 64-bit words ------------------------------------------------------------------------------
DRB_DEV void ll_store(unsigned long long* p, uint32_t payload, uint32_t tag) {
  const unsigned long long v = ((unsigned long long)tag << 32) | payload;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// The same word into every replica (p points into replica 0).
DRB_DEV void ll_store_all(unsigned long long* p, int reps, uint32_t payload, uint32_t tag) {
  for (int r = 0; r < reps; ++r) ll_store(p + (size_t)r * COPY_WORDS, payload, tag);
}
DRB_DEV void ll_load2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
DRB_DEV unsigned long long ll_load1(const unsigned long long* p) {
  unsigned long long a;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  return a;
}

// What a poll does when its data has not arrived. A hand-over completes within a few round trips through L2 and a
// sleeping warp wakes up late (measured: any sleep between retries costs more than a microsecond per layer), so
// retries go out back to back; what keeps them cheap is that every poll asks for whole cache lines. Only a wait
// that has already lasted milliseconds backs off. Every so often the poll looks whether this block or any other
// has given up. Returns true when the caller must stop waiting.
DRB_DEV bool poll_failed(unsigned it, unsigned limit, volatile int* abort_flag) {
  if (it >= limit) {
    atomicMax(&g_drb_error, (unsigned)DRB_ERR_GRID_WAIT);
    *abort_flag = 1;
    return true;
  }
  if (it > 8192) __nanosleep(400);
  if ((it & 1023u) == 1023u && (*abort_flag || *reinterpret_cast<volatile unsigned*>(&g_drb_error) != 0u)) {
    *abort_flag = 1;
    return true;
  }
  return false;
}

// Waits for NV consecutive 16-byte pieces (two tagged words each) at p and returns their 2 NV payloads.
// Pieces that have arrived are not requested again. On give-up the missing payloads are zero.
template <int NV>
DRB_DEV void ll_poll(const unsigned long long* p, uint32_t tag, uint32_t (&out)[2 * NV], unsigned limit, volatile int* abort_flag) {
  unsigned need = (1u << NV) - 1u;
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) out[i] = 0u;
  if (*abort_flag) return;
  unsigned long long ra[2 * NV];
  unsigned ma = 0u;
  auto issue = [&](unsigned long long (&r)[2 * NV], unsigned& m) {
    m = need;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if ((m >> i) & 1u) ll_load2(p + 2 * i, r[2 * i], r[2 * i + 1]);
  };
  auto take = [&](const unsigned long long (&r)[2 * NV], unsigned m) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (((m & need) >> i) & 1u) {
        if ((uint32_t)(r[2 * i] >> 32) == tag && (uint32_t)(r[2 * i + 1] >> 32) == tag) {
          out[2 * i] = (uint32_t)r[2 * i], out[2 * i + 1] = (uint32_t)r[2 * i + 1];
          need &= ~(1u << i);
        }
      }
  };
  issue(ra, ma);
  for (unsigned it = 0;; ++it) {
    take(ra, ma);
    if (need == 0u) break;
    issue(ra, ma);
    if (poll_failed(it, limit, abort_flag)) break;
  }
}

DRB_DEV uint32_t ll_poll1(const unsigned long long* p, uint32_t tag, unsigned limit, volatile int* abort_flag) {
  if (*abort_flag) return 0u;
  unsigned long long a = ll_load1(p);
  for (unsigned it = 0;; ++it) {
    if ((uint32_t)(a >> 32) == tag) return (uint32_t)a;
    a = ll_load1(p);
    if (poll_failed(it, limit, abort_flag)) return 0u;
  }
}

// The whole warp waits for NP consecutive 16-byte pieces at p and writes their 2 NP payload words to `pay` (shared
// memory, private to the warp). Lane i asks for pieces i, i + 32, ...: every request of the warp covers whole cache
// lines, a quarter of the requests that lanes fetching their own scattered pieces would make.
template <int NP>
DRB_DEV void ll_poll_warp(const unsigned long long* p, uint32_t tag, uint32_t* pay, int lane, unsigned limit, volatile int* abort_flag) {
  constexpr int PER = (NP + 31) / 32;
  unsigned need = 0u;
#pragma unroll
  for (int i = 0; i < PER; ++i)
    if (lane + 32 * i < NP) need |= 1u << i;
  const bool skip = *abort_flag != 0;
  unsigned long long ra[2 * PER];
  unsigned ma = 0u;
  auto issue = [&](unsigned long long (&r)[2 * PER], unsigned& m) {
    m = need;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if ((m >> i) & 1u) ll_load2(p + 2 * (lane + 32 * i), r[2 * i], r[2 * i + 1]);
  };
  auto take = [&](const unsigned long long (&r)[2 * PER], unsigned m) {
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (((m & need) >> i) & 1u) {
        if ((uint32_t)(r[2 * i] >> 32) == tag && (uint32_t)(r[2 * i + 1] >> 32) == tag) {
          *reinterpret_cast<uint2*>(pay + 2 * (lane + 32 * i)) = make_uint2((uint32_t)r[2 * i], (uint32_t)r[2 * i + 1]);
          need &= ~(1u << i);
        }
      }
  };
  if (!skip) {
    issue(ra, ma);
    for (unsigned it = 0;; ++it) {
      take(ra, ma);
      if (!__any_sync(0xffffffffu, need != 0u)) break;
      issue(ra, ma);
      if (poll_failed(it, limit, abort_flag)) break;  // the same decision in every lane
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i)
    if ((need >> i) & 1u) *reinterpret_cast<uint2*>(pay + 2 * (lane + 32 * i)) = make_uint2(0u, 0u);
  __syncwarp();
}

// mbarrier wait that honours the abort flag; bounded like the polls, and without sleeping while the wait is short.
DRB_DEV void wait_full(uint64_t* bar, unsigned parity, unsigned limit, volatile int* abort_flag) {
  if (*abort_flag) return;
  for (unsigned it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return;
    if (it >= limit) {
      atomicMax(&g_drb_error, (unsigned)DRB_ERR_FULL_WAIT);
      *abort_flag = 1;
      return;
    }
    if (it > 8192) __nanosleep(400);
    if ((it & 1023u) == 1023u && *abort_flag) return;
  }
}

// One warp turns 32 values (lane = input index) into the 26 tagged words of a routed activation block, in every replica.
DRB_DEV void publish_block32(float v, unsigned long long* dst, int reps, uint32_t tag, int lane) {
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
  // lane 8 j + i (j < 3, i < 8) stores limb word j of input group i; lane 24 the delta, lane 25 the sum
  const uint32_t sel = lane < 8 ? 0x0040u : lane < 16 ? 0x0051u : 0x0062u;
  uint32_t w = prmt(prmt(t0, t1, sel), prmt(t2, t3, sel), 0x5410u);
  if (lane == 24) w = __float_as_uint(delta);
  if (lane == 25) w = __float_as_uint(sum);
  if (lane < ACT_R_WORDS) ll_store_all(dst + lane, reps, w, tag);
}

// Each half-warp turns 16 values (lane & 15 = input index) into the 14 tagged words of a shared-expert block
// at dst + 14 * half, in every replica.
DRB_DEV void publish_block16x2(float v, unsigned long long* dst, int reps, uint32_t tag, int lane) {
  float m = fabsf(v);
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
  int l0, l1, l2;
  limbs3(__float2int_rn(v * (1.f / delta)), l0, l1, l2);
  const uint32_t pack = (uint32_t)(l0 & 0xff) | ((uint32_t)(l1 & 0xff) << 8) | ((uint32_t)(l2 & 0xff) << 16);
  // lane 16 h + 4 j + q (j < 3, q < 4) stores limb word j of inputs 4 q .. 4 q + 3 of half h; lane 16 h + 12 the delta, 16 h + 13 a pad
  const int h = lane >> 4, li = lane & 15, q = li & 3;
  const int base = 16 * h + 4 * q;
  const uint32_t t0 = __shfl_sync(0xffffffffu, pack, base), t1 = __shfl_sync(0xffffffffu, pack, base + 1);
  const uint32_t t2 = __shfl_sync(0xffffffffu, pack, base + 2), t3 = __shfl_sync(0xffffffffu, pack, base + 3);
  const uint32_t sel = li < 4 ? 0x0040u : li < 8 ? 0x0051u : 0x0062u;
  uint32_t w = prmt(prmt(t0, t1, sel), prmt(t2, t3, sel), 0x5410u);
  if (li == 12) w = __float_as_uint(delta);
  if (li == 13) w = 0u;
  if (li < ACT_S_WORDS) ll_store_all(dst + h * ACT_S_WORDS + li, reps, w, tag);
}

// The down rows are requested once this part of the block's gate/up rows has landed: asked for at once they
// compete with the gate/up rows for the memory queue, and the gate/up rows are needed first.
constexpr int DOWN_AFTER_PART = 3;

__global__ void __launch_bounds__(THREADS, 1)
    k_moe_stack(const drb_moe_layer* __restrict__ layers, int n_layers, float* x, Copy* ws, int reps, int E, float eps,
                int* __restrict__ idx_trace, float* __restrict__ wts_trace, unsigned poll_limit) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* qx = dyn + CTL_BYTES;
  unsigned char* rw = qx + QX_BYTES;
  unsigned char* qs = rw + RW_BYTES;
  unsigned char* pa = qs + QS_BYTES;
  unsigned char* gst = pa + PA_BYTES;
  unsigned char* dst = gst + GU_STAGE_S;
  volatile int* abort_flag = &ctl.abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  const bool has_units = b < UNIT_BLOCKS;
  const bool shared_blk = b >= ROUTED_UB && b < UNIT_BLOCKS;
  const bool routed_blk = b < ROUTED_UB;
  const int j0 = shared_blk ? (b - ROUTED_UB) * UNITS : (b % (I / UNITS)) * UNITS;  // first unit of the block
  const int n0 = (int)((long long)H * b / G), n1 = (int)((long long)H * (b + 1) / G), nr = n1 - n0;  // down rows
  const int rrow0 = 2 * b, nrr = max(0, min(2, E + 1 - rrow0));                                     // router rows
  const bool needs_x = has_units || nrr > 0;
  const Copy* mine = ws + (b % reps);  // the replica this block reads

  if (threadIdx.x == 0) {
    for (int q = 0; q < PARTS; ++q) mbar_init(&ctl.gfull[q], 1);
    mbar_init(&ctl.dfull_r, 1);
    mbar_init(&ctl.dfull_s, 1);
    mbar_init(&ctl.rfull, 1);
    ctl.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // =========================== producer warp ===========================
    auto issue_router = [&](const drb_moe_layer& L) {
      if (lane == 0 && nrr > 0) {
        mbar_expect_tx(&ctl.rfull, (unsigned)(nrr * H * 2));
        bulk_g2s(rw, static_cast<const unsigned char*>(L.router) + (size_t)rrow0 * H * 2, (unsigned)(nrr * H * 2), &ctl.rfull);
      }
    };
    // lane 4 q + c requests copy c (gate rows, up rows, gate scales, up scales) of part q
    auto issue_shared_gu = [&](const drb_moe_layer& L) {
      if (!shared_blk) return;
      const int q = lane >> 2, c = lane & 3;
      if (q >= PARTS) return;
      if (c == 0) mbar_expect_tx(&ctl.gfull[q], (unsigned)(2 * PU * (H + SSROW)));
      __syncwarp(0x0000ffffu);
      const unsigned char* shq = static_cast<const unsigned char*>(L.sgu_q);
      const unsigned char* sp = static_cast<const unsigned char*>(L.sgu_s);
      const int u0 = j0 + q * PU, l0 = q * PU;
      if (c == 0) bulk_g2s(gst + (size_t)l0 * H, shq + (size_t)u0 * H, PU * H, &ctl.gfull[q]);
      else if (c == 1) bulk_g2s(gst + (size_t)(UNITS + l0) * H, shq + ((size_t)I + u0) * H, PU * H, &ctl.gfull[q]);
      else if (c == 2) bulk_g2s(gst + (size_t)2 * UNITS * H + l0 * SSROW, sp + (size_t)u0 * SSROW, PU * SSROW, &ctl.gfull[q]);
      else bulk_g2s(gst + (size_t)2 * UNITS * H + (UNITS + l0) * SSROW, sp + ((size_t)I + u0) * SSROW, PU * SSROW, &ctl.gfull[q]);
    };
    auto issue_shared_dn = [&](const drb_moe_layer& L) {
      if (lane == 0 && nr > 0) {
        mbar_expect_tx(&ctl.dfull_s, (unsigned)(nr * I));
        bulk_g2s(dst + TOPK * D_EXPERT, static_cast<const unsigned char*>(L.sd_q) + (size_t)n0 * I, (unsigned)(nr * I), &ctl.dfull_s);
      }
    };
    // Needs ctl.idx (the gate/up rows are requested by consumer warp 0, which finishes the selection). Lanes 16..23: the down rows of expert slot lane - 16.
    auto issue_routed_dn = [&](const drb_moe_layer& L) {
      if (nr > 0 && lane >= 16 && lane < 16 + TOPK) {
        if (lane == 16) mbar_expect_tx(&ctl.dfull_r, (unsigned)(nr * TOPK * (DQROW + DSMROW)));
        __syncwarp(0x00ff0000u);
        const int k = lane - 16;
        const size_t row = (size_t)ctl.idx[k] * H + n0;
        bulk_g2s(dst + k * D_EXPERT, static_cast<const unsigned char*>(L.d_q) + row * DQROW, (unsigned)(nr * DQROW), &ctl.dfull_r);
        bulk_g2s(dst + k * D_EXPERT + RT * DQROW, static_cast<const unsigned char*>(L.d_sm) + row * DSMROW,
                 (unsigned)(nr * DSMROW), &ctl.dfull_r);
      }
    };

    drb_moe_layer Lc = layers[0], Ln = Lc;
    issue_router(Lc);
    issue_shared_gu(Lc);
    issue_shared_dn(Lc);
    for (int l = 0; l < n_layers; ++l) {
      const bool more = l + 1 < n_layers;
      if (more) Ln = layers[l + 1];  // in registers before the routing arrives
      bar_sync<256 + 32>(BAR_IDX);   // the routing of layer l is in ctl
      // The gate/up rows are what the layer waits for; the down rows are needed a hand-over later. Requested together
      // they share the memory system and delay the activations, so they follow once part of the gate/up rows is here.
      if (routed_blk) wait_full(&ctl.gfull[DOWN_AFTER_PART], (unsigned)l & 1u, poll_limit, abort_flag);
      issue_routed_dn(Lc);
      if (nrr > 0) {
        bar_sync<64 + 32>(BAR_RT);
        if (more) issue_router(Ln);
      }
      bar_sync<THREADS>(BAR_GU);
      if (more) issue_shared_gu(Ln);
      bar_sync<THREADS>(BAR_DN);
      if (more) issue_shared_dn(Ln);
      Lc = Ln;
    }
    return;
  }

  // =========================== consumer warps ===========================
  const int t = threadIdx.x;
  float xres = (t < nr) ? __ldcg(x + n0 + t) : 0.f;  // the residual of this thread's output row, carried in a register
  // Warp w fetches the shared expert's activation blocks 2w, 2w + 1 into shared memory (7 pieces each).
  auto fetch_shared_act = [&](uint32_t tag) {
    if (lane < 14) {
      const int sb = 2 * warp + lane / 7, piece = lane % 7;
      uint32_t o[2];
      ll_poll<1>(mine->act_s + (size_t)sb * ACT_S_WORDS + 2 * piece, tag, o, poll_limit, abort_flag);
      *reinterpret_cast<uint2*>(qs + (size_t)sb * QB16_BYTES + piece * 8) = make_uint2(o[0], o[1]);
    }
  };
  // Constants of the coming layer are fetched a layer ahead: a pointer out of the layer table and then the value
  // behind it are two dependent trips to memory, which would otherwise open every layer.
  const unsigned char* guq_next = static_cast<const unsigned char*>(layers[0].gu_q);
  const unsigned char* gusm_next = static_cast<const unsigned char*>(layers[0].gu_sm);
  const float* pn_next = static_cast<const float*>(layers[0].post_norm);
  const __half* sds_next = static_cast<const __half*>(layers[0].sd_s);
  float4 wv_next = needs_x ? reinterpret_cast<const float4*>(pn_next)[t] : make_float4(0.f, 0.f, 0.f, 0.f);
  float ssc_next = warp < nr ? __half2float(__ldg(sds_next + (size_t)(n0 + warp) * (I / 128) + (lane >> 3))) : 0.f;
  for (int l = 0; l < n_layers; ++l) {
    const uint32_t tag = (uint32_t)l + 1u;
    const unsigned par = (unsigned)l & 1u;
    const float4 wv = wv_next;
    const float ssc = ssc_next;
    const unsigned char* guq_cur = guq_next;
    const unsigned char* gusm_cur = gusm_next;
    if (l + 1 < n_layers) {
      guq_next = static_cast<const unsigned char*>(layers[l + 1].gu_q);
      gusm_next = static_cast<const unsigned char*>(layers[l + 1].gu_sm);
      pn_next = static_cast<const float*>(layers[l + 1].post_norm);
      sds_next = static_cast<const __half*>(layers[l + 1].sd_s);
    }

    // ---- the hidden state: sum of squares and this block's two router rows in one pass, then the limb blocks.
    // The logits are linear in the hidden state, so the rows are multiplied with y * norm weight as it arrives and
    // the 1 / rms factor is applied to the two sums: the routing does not wait for a second pass over x.
    if (needs_x) {
      if (nrr > 0) wait_full(&ctl.rfull, par, poll_limit, abort_flag);
      float4 xv;
      if (l == 0) {
        xv = __ldcg(reinterpret_cast<const float4*>(x) + t);
      } else {
        uint32_t o[4];
        ll_poll<2>(mine->y + 4 * t, tag - 1u, o, poll_limit, abort_flag);
        xv = make_float4(__uint_as_float(o[0]), __uint_as_float(o[1]), __uint_as_float(o[2]), __uint_as_float(o[3]));
      }
      const float4 xw = make_float4(xv.x * wv.x, xv.y * wv.y, xv.z * wv.z, xv.w * wv.w);
      float v[4] = {xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w, 0.f, 0.f, 0.f};
      if (nrr > 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint2 w = *reinterpret_cast<const uint2*>(rw + (size_t)r * H * 2 + 8 * t);
          v[1 + r] = (xw.x * __uint_as_float(w.x << 16) + xw.y * __uint_as_float(w.x & 0xffff0000u)) +
                     (xw.z * __uint_as_float(w.y << 16) + xw.w * __uint_as_float(w.y & 0xffff0000u));
        }
      }
      {
        const bool hi16 = lane & 16, hi8 = lane & 8;
        const float r0 = (hi16 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[0] : v[2], 16);
        const float r1 = (hi16 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? v[1] : v[3], 16);
        float s = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        // lanes 0..7 carry v[0], 8..15 v[1], 16..23 v[2]
        if ((lane & 7) == 0 && lane < 24) ctl.red[lane >> 3][warp] = s;
      }
      bar_sync<NT>(BAR_CONS);
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < CW; ++w) tot += ctl.red[0][w];
      const float inv = rsqrtf(tot / H + eps);
      if (t < nrr) {
        float u = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) u += ctl.red[1 + t][w];
        ll_store_all(ws->logits + rrow0 + t, reps, __float_as_uint(u * inv), tag);
      }
      if (warp < 2 && nrr > 0) bar_arrive<64 + 32>(BAR_RT);  // every warp read its part of the rows before the barrier above
      if (has_units) {
        quant_store_eo(qx, t, make_float4(xw.x * inv, xw.y * inv, xw.z * inv, xw.w * inv), true);
        bar_sync<NT>(BAR_CONS);
      }
    }

    // ---- warps 0..7 of every block derive the routing from the E + 1 logits. A shared-expert block does its gate/up
    // rows first: they do not depend on the routing, and every other block needs their activations.
    //
    // What the layer waits for is the request for the chosen experts' rows, so the selection is made on the logits
    // alone (softmax is monotone: the eight largest logits are the eight largest probabilities) and warp 0, which
    // finishes the selection, requests this block's gate/up rows itself. The probabilities and weights follow while
    // the rows are on their way. Selection: the per-warp maxima bound it from below (eight entries are at least as
    // large as the smallest of eight warp maxima), the few entries at or above the bound are ranked against each
    // other by warp 0 with shuffles, ties to the lower index. An entry whose probability merely rounds to that of a
    // larger logit is never preferred to it, which is the one place where this differs from ranking rounded
    // probabilities.
    auto derive_routing = [&]() {
      // the shared expert's gate logit is fetched by a thread that has no logit of its own to wait for (two waits in
      // one thread are two round trips); it is read after the next barrier of all consumers
      if (t == 256) ctl.sgate = __uint_as_float(ll_poll1(mine->logits + E, tag, poll_limit, abort_flag));
      if (warp >= 8) return;
      router::TopkSmem& tk = ctl.tk;
      const bool valid = t < E;
      float v = -INFINITY;
      if (valid) v = __uint_as_float(ll_poll1(mine->logits + t, tag, poll_limit, abort_flag));
      const unsigned vb = __float_as_uint(v);
      const unsigned ord = (vb & 0x80000000u) ? ~vb : (vb | 0x80000000u);  // orders like the floats
      const unsigned wmax = __reduce_max_sync(0xffffffffu, ord);
      if (lane == 0) tk.ured[warp] = wmax;
      bar_sync<256>(BAR_TOPK);
      const int nvalid = (E + 31) >> 5;  // warps that hold valid entries
      unsigned mo = tk.ured[0], lo = tk.ured[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        const unsigned u = tk.ured[w];
        mo = max(mo, u);
        if (w < nvalid) lo = min(lo, u);
      }
      if (nvalid < TOPK) lo = 0u;  // fewer than eight maxima: every valid entry stays in
      const bool cand = valid && ord >= lo;
      const unsigned bal = __ballot_sync(0xffffffffu, cand);
      if (cand) tk.comp[warp * router::MAX_TOPK + __popc(bal & ((1u << lane) - 1u))] = ((unsigned long long)ord << 32) | (unsigned)(~t);
      if (lane == 0) tk.cnt[warp] = __popc(bal);
      bar_sync<256>(BAR_TOPK);
      // the softmax denominator does not depend on the selection and is off the path to the requests:
      // same reduction tree as dr_router_topk
      const float m = router::ord_to_float(mo);
      if (warp != 0) {
        bar_arrive<256 + 32>(BAR_IDX);
        const float wsum = warp_sum(valid ? expf(v - m) : 0.f);
        if (lane == 0) tk.red[warp] = wsum;
        bar_sync<256>(BAR_TOPK);
        return;
      }
      int off[9];
      off[0] = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) off[w + 1] = off[w] + tk.cnt[w];
      const int n = off[8];
      auto fetch = [&](int i) {  // survivor i sits in warp w's segment at position i - off[w]; list order is index order
        int w = 0, ow = 0;
#pragma unroll
        for (int q = 1; q < 8; ++q) {
          const bool past = i >= off[q];
          w += past ? 1 : 0;
          ow = past ? off[q] : ow;
        }
        return tk.comp[w * router::MAX_TOPK + (i - ow)];
      };
      if (n <= 32) {
        const unsigned long long c = lane < n ? fetch(lane) : 0ull;
        const unsigned k = (unsigned)(c >> 32);
        int r = 0;
#pragma unroll
        for (int o = 1; o < 32; ++o) {
          const int src = (lane + o) & 31;
          const unsigned ko = __shfl_sync(0xffffffffu, k, src);
          r += (ko > k || (ko == k && src < lane)) ? 1 : 0;
        }
        if (lane < n && r < TOPK) ctl.idx[r] = (int)(~(unsigned)c), tk.ukey[r] = k;
      } else {
        for (int i = lane; i < n; i += 32) {  // many ties at the bound: rank against the whole list
          const unsigned long long c = fetch(i);
          int g = 0;
#pragma unroll
          for (int w2 = 0; w2 < 8; ++w2) {
            const int c2 = off[w2 + 1] - off[w2];
            for (int j = 0; j < c2; ++j) g += tk.comp[w2 * router::MAX_TOPK + j] > c ? 1 : 0;
          }
          if (g < TOPK) ctl.idx[g] = (int)(~(unsigned)c), tk.ukey[g] = (unsigned)(c >> 32);
        }
      }
      __syncwarp();
      // this block's gate/up rows: lane 4 q + c requests copy c (gate rows, up rows, gate scales, up scales) of part q
      if (routed_blk && lane < 4 * PARTS) {
        const int q = lane >> 2, c = lane & 3;
        if (c == 0) mbar_expect_tx(&ctl.gfull[q], (unsigned)(2 * PU * (QROW + SMROW)));
        __syncwarp(0x0000ffffu);
        const size_t ek = (size_t)ctl.idx[b / (I / UNITS)];
        const unsigned char* qp = guq_cur + ek * (2 * I) * QROW;
        const unsigned char* smp = gusm_cur + ek * (2 * I) * SMROW;
        const int u0 = j0 + q * PU, l0 = q * PU;
        if (c == 0) bulk_g2s(gst + (size_t)l0 * QROW, qp + (size_t)u0 * QROW, PU * QROW, &ctl.gfull[q]);
        else if (c == 1) bulk_g2s(gst + (size_t)(UNITS + l0) * QROW, qp + ((size_t)I + u0) * QROW, PU * QROW, &ctl.gfull[q]);
        else if (c == 2) bulk_g2s(gst + (size_t)2 * UNITS * QROW + l0 * SMROW, smp + (size_t)u0 * SMROW, PU * SMROW, &ctl.gfull[q]);
        else bulk_g2s(gst + (size_t)2 * UNITS * QROW + (UNITS + l0) * SMROW, smp + ((size_t)I + u0) * SMROW, PU * SMROW, &ctl.gfull[q]);
      }
      bar_arrive<256 + 32>(BAR_IDX);  // the producer warp requests the down rows
      {
        const float wsum = warp_sum(valid ? expf(v - m) : 0.f);
        if (lane == 0) tk.red[0] = wsum;
      }
      bar_sync<256>(BAR_TOPK);
      // weights: p = exp(v - m) / z of the chosen eight, renormalised over their sum taken in the order
      // "larger probability, then lower index" (kernels/drama.cu:397-435 of the reference)
      const float z = ((tk.red[0] + tk.red[4]) + (tk.red[2] + tk.red[6])) + ((tk.red[1] + tk.red[5]) + (tk.red[3] + tk.red[7]));
      const int sl = lane & (TOPK - 1);
      const float pj = expf(router::ord_to_float(tk.ukey[sl]) - m) / z;
      const int ej = ctl.idx[sl];
      int rj = 0;
#pragma unroll
      for (int o = 1; o < TOPK; ++o) {
        const int src = (lane & ~(TOPK - 1)) | ((sl + o) & (TOPK - 1));
        const float po = __shfl_sync(0xffffffffu, pj, src);
        const int eo = __shfl_sync(0xffffffffu, ej, src);
        rj += (po > pj || (po == pj && eo < ej)) ? 1 : 0;
      }
      if (lane < TOPK) tk.top[rj] = pj;
      __syncwarp();
      float total = 0.f;
#pragma unroll
      for (int k2 = 0; k2 < TOPK; ++k2) total += tk.top[k2];
      if (lane < TOPK) {
        ctl.wts[lane] = pj / total;  // per slot; the slots are in logit order
        if (b == 0) {                // the routing as the reference reports it
          if (idx_trace) idx_trace[l * TOPK + rj] = ej;
          if (wts_trace) wts_trace[l * TOPK + rj] = pj / total;
        }
      }
    };
    if (!shared_blk) derive_routing();

    // ---- gate/up + SwiGLU on this block's 32 units
    if (has_units) {
      // This lane owns k in [32 lane, +32) and [1024 + 32 lane, +32).
      QAct<32, true> x0, x1;
      float X0, X1;
      qact_load(x0, X0, qx + (size_t)lane * QB32_BYTES);
      qact_load(x1, X1, qx + (size_t)(32 + lane) * QB32_BYTES);
      float v[4];  // v[2i] = gate, v[2i + 1] = up partial sums of unit warp + 16 i
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int u = warp + CW * i;
        // Between its two units a routed block picks up the shared expert's activations: they were published while this
        // block waited for its rows (a shared block fetches them after it has published its own).
        if (i == 1 && routed_blk) fetch_shared_act(tag);
        wait_full(&ctl.gfull[u / PU], par, poll_limit, abort_flag);
        if (shared_blk) {
          const uint4* gr = reinterpret_cast<const uint4*>(gst + (size_t)u * H);
          const uint4* ur = reinterpret_cast<const uint4*>(gst + (size_t)(UNITS + u) * H);
          const __half* gs = reinterpret_cast<const __half*>(gst + (size_t)2 * UNITS * H + (size_t)u * SSROW);
          const __half* us = reinterpret_cast<const __half*>(gst + (size_t)2 * UNITS * H + (size_t)(UNITS + u) * SSROW);
          v[2 * i] = __half2float(gs[lane >> 2]) * x0.delta * dot32_q8_eo(gr[2 * lane], gr[2 * lane + 1], x0, 0) +
                     __half2float(gs[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(gr[64 + 2 * lane], gr[64 + 2 * lane + 1], x1, 0);
          v[2 * i + 1] = __half2float(us[lane >> 2]) * x0.delta * dot32_q8_eo(ur[2 * lane], ur[2 * lane + 1], x0, 0) +
                         __half2float(us[8 + (lane >> 2)]) * x1.delta * dot32_q8_eo(ur[64 + 2 * lane], ur[64 + 2 * lane + 1], x1, 0);
        } else {
          const uint4* gr = reinterpret_cast<const uint4*>(gst + (size_t)u * QROW);
          const uint4* ur = reinterpret_cast<const uint4*>(gst + (size_t)(UNITS + u) * QROW);
          const __half2* gs = reinterpret_cast<const __half2*>(gst + (size_t)2 * UNITS * QROW + (size_t)u * SMROW);
          const __half2* us = reinterpret_cast<const __half2*>(gst + (size_t)2 * UNITS * QROW + (size_t)(UNITS + u) * SMROW);
          // w = s q + m: sum_k w x = s delta sum(q n) + m sum(x) per 64-group; chunk c belongs to group c / 2.
          const float2 g0 = __half22float2(gs[lane >> 1]), g1 = __half22float2(gs[16 + (lane >> 1)]);
          const float2 u0 = __half22float2(us[lane >> 1]), u1 = __half22float2(us[16 + (lane >> 1)]);
          v[2 * i] = g0.x * x0.delta * dot32_q4_i(gr[lane], x0, 0) + g0.y * X0 + g1.x * x1.delta * dot32_q4_i(gr[32 + lane], x1, 0) + g1.y * X1;
          v[2 * i + 1] = u0.x * x0.delta * dot32_q4_i(ur[lane], x0, 0) + u0.y * X0 + u1.x * x1.delta * dot32_q4_i(ur[32 + lane], x1, 0) + u1.y * X1;
        }
      }
      bar_arrive<THREADS>(BAR_GU);  // nothing of the stage is read after this point
      // Fold the four per-lane sums into one reduction.
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
      bar_sync<NT>(BAR_CONS);
      if (warp == 0) {
        const float a = ctl.actv[lane];
        if (shared_blk) publish_block16x2(a, ws->act_s + (size_t)(b - ROUTED_UB) * 2 * ACT_S_WORDS, reps, tag, lane);
        else publish_block32(a, ws->act_r + (size_t)b * ACT_R_WORDS, reps, tag, lane);
      }
    } else {
      bar_arrive<THREADS>(BAR_GU);
    }
    if (shared_blk) derive_routing();

    // ---- down + combine on this block's rows
    {
      if (!routed_blk) {  // a routed block fetched them between its two units; the barrier there made them visible
        fetch_shared_act(tag);
        bar_sync<NT>(BAR_CONS);
      }
      if (l + 1 < n_layers) {  // the next layer's constants, needed a layer from now
        if (needs_x) wv_next = reinterpret_cast<const float4*>(pn_next)[t];
        if (warp < nr) ssc_next = __half2float(__ldg(sds_next + (size_t)(n0 + warp) * (I / 128) + (lane >> 3)));
      }
      QAct<16, false> sq;  // the shared expert: the whole warp per row, lane = 16-byte chunk of 16 int8
      qact_load(sq, qs + (size_t)lane * QB16_BYTES);
      // routed: warp (ke, kh) covers inputs [256 kh, +256) of expert slot ke; lane (rsub, c): row 4 pass + rsub, 16-byte chunk 8 kh + c
      const int ke = warp & (TOPK - 1), kh = warp >> 3;
      const int c = lane & 7, rsub = lane >> 3;
      const int chunk = kh * 8 + c;
      QAct<32, true> aq;
      float A;
      {
        // the warp's eight blocks are contiguous: fetched together, then every lane takes the 26 words of its block
        uint32_t* mypa = reinterpret_cast<uint32_t*>(pa + (size_t)warp * PA_WARP_BYTES);
        ll_poll_warp<8 * ACT_R_WORDS / 2>(mine->act_r + (size_t)(ke * (I / 32) + kh * 8) * ACT_R_WORDS, tag, mypa, lane, poll_limit, abort_flag);
        const uint2* src = reinterpret_cast<const uint2*>(mypa + c * ACT_R_WORDS);
        uint32_t o[ACT_R_WORDS];
#pragma unroll
        for (int i = 0; i < ACT_R_WORDS / 2; ++i) {
          const uint2 w2 = src[i];
          o[2 * i] = w2.x, o[2 * i + 1] = w2.y;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 3; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) aq.l[j][i] = o[j * 8 + i];
        aq.delta = __uint_as_float(o[24]);
        A = __uint_as_float(o[25]);
      }
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      float s_sh = 0.f;
      if (nr > 0) {
        wait_full(&ctl.dfull_r, par, poll_limit, abort_flag);
        const unsigned char* eq = dst + ke * D_EXPERT;
        const unsigned char* esm = eq + RT * DQROW;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int lr = 4 * p + rsub;
          if (lr < nr) {
            const uint4 w = *reinterpret_cast<const uint4*>(eq + (size_t)lr * DQROW + 16 * chunk);
            const float2 sm = __half22float2(*reinterpret_cast<const __half2*>(esm + (size_t)lr * DSMROW + 4 * (chunk >> 1)));
            v[p] = sm.x * aq.delta * dot32_q4_i(w, aq, 0) + sm.y * A;
          }
        }
        if (warp < nr) {
          wait_full(&ctl.dfull_s, par, poll_limit, abort_flag);
          s_sh = ssc * sq.delta * dot16_q8_i(*reinterpret_cast<const uint4*>(dst + TOPK * D_EXPERT + (size_t)warp * I + 16 * lane), sq, 0);
        }
      }
      bar_arrive<THREADS>(BAR_DN);  // nothing of the stage is read after this point
      {
        // Fold the four sums (each to be reduced over the 8 lanes of a row group) into one reduction.
        const bool hi4 = lane & 4, hi2 = lane & 2;
        const float r0 = (hi4 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi4 ? v[0] : v[2], 4);
        const float r1 = (hi4 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi4 ? v[1] : v[3], 4);
        float s = (hi2 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi2 ? r0 : r1, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        const int p = (hi4 ? 2 : 0) + (hi2 ? 1 : 0);
        const int lr = 4 * p + rsub;
        if ((lane & 1) == 0 && lr < nr) ctl.part[ke][kh][lr] = s;
      }
      s_sh = warp_sum(s_sh);
      if (lane == 0 && warp < nr) ctl.part_s[warp] = s_sh;
      bar_sync<NT>(BAR_CONS);
      if (t < nr) {
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < TOPK; ++k) acc += ctl.wts[k] * (ctl.part[k][0][t] + ctl.part[k][1][t]);
        const float yn = xres + sigmoid_f(ctl.sgate) * ctl.part_s[t] + acc;
        xres = yn;
        if (l + 1 < n_layers) ll_store_all(ws->y + n0 + t, reps, __float_as_uint(yn), tag);
        else x[n0 + t] = yn;
      }
    }
  }
}

static cudaError_t configure_all() {
  cudaError_t e = cudaFuncSetAttribute(k_moe_stack, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return drb_carveout(k_moe_stack);
}

// One block whose waits cannot be satisfied: nothing ever arrives at its mbarrier, nothing ever tags `word`. Each
// wait gives up after `limit` polls, records its code and lets the kernel run to its end, which is what the host
// observes through drb_device_error(). which = 1: the copy wait of the per-layer kernels (mbar_wait); 2: the copy wait
// of the persistent kernel (wait_full); 3: its tagged-word polls, by one thread and then by whole warps, the later
// ones returning at once because the block has already given up.
__global__ void __launch_bounds__(64, 1) k_test_waits(int which, unsigned limit, const unsigned long long* word, unsigned* polls_after) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  __shared__ __align__(16) uint32_t pay[2 * 32];  // ll_poll_warp stores payload pairs as 8-byte words
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    abort_word = 0;
  }
  __syncthreads();
  volatile int* abort_flag = &abort_word;
  if (which == 1) {
    if (threadIdx.x == 0) mbar_wait(&bar, 0, DRB_ERR_FULL_WAIT, limit);
  } else if (which == 2) {
    if (threadIdx.x == 0) wait_full(&bar, 0, limit, abort_flag);
    __syncthreads();
    wait_full(&bar, 0, limit, abort_flag);  // every thread: returns at once, the block has given up
  } else {
    if (threadIdx.x == 0) ll_poll1(word, 1u, limit, abort_flag);
    __syncthreads();
    const long long t0 = clock64();
    ll_poll_warp<32>(word, 1u, pay + 0, lane, limit, abort_flag);  // returns at once with zero payloads
    if (threadIdx.x == 0 && polls_after) *polls_after = (unsigned)(clock64() - t0) + (pay[0] | pay[1]);
  }
}

constexpr unsigned POLL_LIMIT = 1u << 20;  // about half a second of polling

}  // namespace stack

// Bytes of device workspace drb_moe_stack_decode needs (any contents; every call clears what it uses first).
extern "C" int drb_moe_stack_workspace_bytes(void) { return (int)sizeof(stack::Copy); }

// x <- x + moe_l(rmsnorm(x)) for l = 0 .. n_layers - 1, in place, in one cooperative kernel launch.
// layers: device array of n_layers drb_moe_layer. workspace: drb_moe_stack_workspace_bytes() bytes of
// device memory, 256-byte aligned. idx_trace / wts_trace: optional device arrays [n_layers, topk]
// receiving every layer's routing (NULL to skip). Only h = 2048, i = 512, topk = 8, e <= 256, and a
// device with at least 144 multiprocessors are supported (-1 otherwise). Capturable in a graph.
// Calls that share a workspace must not overlap on the GPU.
extern "C" int drb_moe_stack_decode(const drb_moe_layer* layers, int n_layers, float* x, void* workspace, int e, int topk,
                                    int h, int i, float eps, int* idx_trace, float* wts_trace, cudaStream_t st) {
  if (h != moe::H || i != moe::I || topk != moe::TOPK || e < topk || e > stack::MAX_E || n_layers < 0) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (dev.sms < stack::MIN_GRID || dev.sms > stack::MAX_GRID) return -1;
  if (n_layers == 0) return 0;
  stack::Copy* ws = static_cast<stack::Copy*>(workspace);
  int reps = 1;  // see Copy
  // tags restart at 1 with every launch, so whatever an earlier launch left must not look valid
  cudaError_t err = cudaMemsetAsync(ws, 0, sizeof(stack::Copy), st);
  if (err != cudaSuccess) return (int)err;
  unsigned limit = stack::POLL_LIMIT;
  void* args[] = {(void*)&layers, (void*)&n_layers, (void*)&x, (void*)&ws, (void*)&reps, (void*)&e, (void*)&eps, (void*)&idx_trace, (void*)&wts_trace, (void*)&limit};
  err = cudaLaunchCooperativeKernel((const void*)stack::k_moe_stack, dim3(dev.sms), dim3(stack::THREADS), args, stack::SMEM_BYTES, st);
  return err == cudaSuccess ? 0 : (int)err;
}

// Test hook (no counterpart in the reference): launches one block whose bounded wait runs out after `limit` polls
// (which: 1 = mbar_wait, 2 = wait_full, 3 = tagged-word polls; word: 512 zeroed bytes of device memory; clocks: a
// device word receiving the clocks the later polls of case 3 took, or NULL). The launch completes normally; the
// code is then read with drb_device_error(). limit <= 65536 (a few milliseconds), else -1.
extern "C" int drb_test_wait_runs_out(int which, unsigned limit, const void* word, unsigned* clocks, cudaStream_t st) {
  if (which < 1 || which > 3 || limit == 0 || limit > 65536u || !word) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  stack::k_test_waits<<<1, 64, 0, st>>>(which, limit, static_cast<const unsigned long long*>(word), clocks);
  return (int)cudaGetLastError();
}
