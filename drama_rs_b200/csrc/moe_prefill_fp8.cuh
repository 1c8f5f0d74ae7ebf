// dr_moe_prefill_fp8 on the native type: the E4M3 weight bytes go from HBM to the tensor cores untouched
// (tiled TMA with the 128-byte swizzle writes the MMA's A operand; tcgen05.mma.kind::f8f6f4), no thread ever
// converts a weight.
//
// The checkpoint's FP8 experts carry one f32 scale per 128 x 128 block (src/model.rs:99-106). A 128-row tile of this
// kernel IS one block row, so over a 128-input chunk the scale is one scalar for the whole tile, and a scalar can
// ride on the other operand: the token tile of chunk kb is B'[t][k] = x[t][k] * s[kb] / c_t, where c_t (one number
// per token and tile, the row's largest magnitude times the tile's largest scale over 256) brings every entry into
// E4M3 range; the accumulator then runs over the whole K without a drain, and the epilogue multiplies by c_t.
// The 8-bit MMA kind takes both operands as 8-bit floats, so B' is written as three E4M3 terms (value, residual,
// residual of the residual: about twelve significant bits, what fp16 operands carry). The three terms of a token are
// three ROWS of the token operand (rows t, 16 + t, 32 + t of a 48-row tile), so one MMA of N = 48 multiplies all three
// and the epilogue adds the three column groups: a third of the MMA issues (an issue costs its thread about 100 cycles, and
// one thread per block issues), for 48 accumulator columns instead of 16.
// A gate/up item holds two accumulators, the 128 gate rows of units [128 mt, +128) and their 128 up rows (two block
// rows with their own scales, hence two B' tiles per chunk); SiLU(gate) * up is formed in the epilogue by the thread
// that holds both.
//
// One block = four prep warps (B' tiles, epilogue), one MMA-issuing warp, a loader warp, a table warp (one item ahead:
// token rows, scales, c_t); two blocks per multiprocessor. Roles meet only on mbarriers; every wait is bounded, and no
// role leaves before the completion arrivals it is owed have landed.
// Work items: (expert, group of up to 16 tokens, 128-row tile), enumerated from the device-side counts.
// Replaces kernels/drama.cu:971-1109 of the reference (k_moe_pf_gate_up_fp8, k_moe_pf_down_fp8).
#pragma once

#include "common.cuh"
#include "moe_prefill_mma.cuh"
#include "moe_prefill_tma.cuh"

namespace pf8 {

using pfmma::f2h_sat;
using pfmma::fence_async_smem;
using pfmma::mma_commit;
using pfmma::smem_desc;
using pfmma::swz_off;
using pfmma::tc_fence_after;
using pfmma::tc_fence_before;
using pfmma::tmem_alloc;
using pfmma::tmem_dealloc;
using pfmma::tmem_ld16;
using pft::tma_load_2d;

constexpr int H = 2048, I = 512;
constexpr int PREP_WARPS = 4, PREPPERS = PREP_WARPS * 32;
constexpr int MMA_WARP = PREP_WARPS, LOAD_WARP = PREP_WARPS + 1, TABLE_WARP = PREP_WARPS + 2;
constexpr int THREADS = PREPPERS + 96;
constexpr int TILE_M = 128;
constexpr int KC = 128;                 // K chunk = one scale block = one 128-byte swizzle row of E4M3
constexpr int NT = 16;                  // tokens per work item = accumulator columns
constexpr int TERMS = 3;
constexpr int A_BYTES = TILE_M * KC;    // 16 KB per accumulator and chunk
constexpr int BT_BYTES = NT * KC;       // 2 KB: one term of one accumulator's token tile
constexpr int MAX_ITEM_SETS = 256;
constexpr int MAX_KB = H / KC;          // 16 scale blocks along the widest K
constexpr int CTL_BYTES = 1024;
constexpr int TAB_SLOT = (2 * NT + 2 * NT + 2 * MAX_KB) * 4 + 16;  // rows, result rows | c (gate, up) | scales (gate, up) | nt
constexpr int NTAB = 2;
constexpr int BASE_BYTES = ((MAX_ITEM_SETS + 1) * 4 + 127) / 128 * 128;

constexpr int NACC = 2;                          // accumulators per item
constexpr int NSA = 2;                           // A stages of 32 KB
constexpr int NSB = 3;                           // B' stages of 12 KB
constexpr int A_STAGE = NACC * A_BYTES;
constexpr int B_STAGE = NACC * TERMS * BT_BYTES;
constexpr size_t SMEM = 1024 + CTL_BYTES + (size_t)NSA * A_STAGE + NSB * B_STAGE + NTAB * TAB_SLOT + BASE_BYTES;
constexpr int NCOL = TERMS * NT;                 // accumulator columns: one group of NT per term
constexpr int TMEM_COLS = 256;                   // two items in flight x two accumulators x 48 columns = 192, rounded up
static_assert(2 * NACC * NCOL <= TMEM_COLS, "tensor memory");
static_assert(SMEM <= 113 * 1024, "two blocks per multiprocessor");

struct Ctl {
  uint64_t afull[4], aempty[4];     // A stage landed (TMA) / its MMAs completed
  uint64_t bfull[3], bempty[3];     // B' stage written (one arrival per prep warp) / its MMAs completed
  uint64_t accfull[2], accfree[2];  // an item's accumulators complete / drained (one arrival per prep warp)
  uint64_t tabfull[NTAB], tabempty[NTAB];
  uint32_t tmem_base;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block");

// kind::f8f6f4, both operands E4M3, fp32 accumulators, K-major, M = 128, N = n.
DRB_DEV uint32_t instr_desc_e4m3(int n) {
  return (1u << 4) /* D = f32 */ | (0u << 7) /* A = E4M3 */ | (0u << 10) /* B = E4M3 */ | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(TILE_M >> 4) << 24);
}
DRB_DEV void mma_e4m3(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// Two floats -> two E4M3 bytes (lo in bits 0..7), round to nearest, saturating; and back, exactly.
DRB_DEV uint32_t f2e4m3x2(float lo, float hi) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
DRB_DEV float2 e4m3x2_to_f2(uint32_t p) {
  uint32_t h2;
  asm("{.reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t;}" : "=r"(h2) : "r"(p));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
// v0, v1 -> three packed E4M3 pairs whose sums approximate them: value, residual, residual of the residual.
DRB_DEV void split3(float v0, float v1, uint32_t (&t)[TERMS]) {
#pragma unroll
  for (int j = 0; j < TERMS; ++j) {
    t[j] = f2e4m3x2(v0, v1);
    const float2 b = e4m3x2_to_f2(t[j]);
    v0 -= b.x, v1 -= b.y;
  }
}

// ---- every token row's largest magnitude ------------------------------------------------------------------------
// One warp per row of xp (bf16 [slots, H]); out[slot] = max |x|. The rows in use end at max_e (offsets[e] + counts[e]).
// Runs ahead of the gate/up kernel, which would otherwise recompute it in every one of a token group's four tiles.
__global__ void __launch_bounds__(256) k_rowmax_bf16(const __nv_bfloat16* __restrict__ xp, const int* __restrict__ offsets,
                                                     const int* __restrict__ counts, int E, float* __restrict__ out) {
  __shared__ int s_total;
  pdl_wait();
  if (threadIdx.x == 0) s_total = 0;
  __syncthreads();
  int end = 0;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = __ldg(counts + e);
    if (c > 0) end = max(end, __ldg(offsets + e) + c);
  }
  end = __reduce_max_sync(0xffffffffu, end);
  if ((threadIdx.x & 31) == 0) atomicMax(&s_total, end);
  __syncthreads();
  const int total = s_total, lane = threadIdx.x & 31;
  constexpr int PER = H / 8 / 32;
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total; row += gridDim.x * (blockDim.x >> 5)) {
    const uint4* p = reinterpret_cast<const uint4*>(xp + (size_t)row * H);
    uint4 v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = __ldg(p + i * 32 + lane);
    uint32_t m = 0u;  // bf16 with the sign bit cleared orders like an integer
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const uint32_t wv[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) m = max(m, max(wv[q] & 0x7fffu, (wv[q] >> 16) & 0x7fffu));
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0) out[row] = __uint_as_float(m << 16);
  }
}

// ---- gate/up + SwiGLU -----------------------------------------------------------------------------------------------
// src = xp bf16 [slots, H] -> dst = act fp16 [slots, I]. tm: gu_w as a tensor map over [E * 2I rows, H bytes], boxes of
// 128 rows x 128 bytes, 128-byte swizzle. S: f32 scales [E, 2I / 128, H / 128]. rmax: k_rowmax_bf16's result.
// An item is (expert, group of up to 16 tokens, 128 units) and runs in 16 steps, one per chunk of K; a step multiplies
// the chunk's box of the units' gate rows into accumulator 0 and the box of their up rows into accumulator 1.
__global__ void __launch_bounds__(THREADS, 2)
    k_gate_up_fp8(const __grid_constant__ CUtensorMap tm, const float* __restrict__ S, const __nv_bfloat16* __restrict__ src,
                  const float* __restrict__ rmax, __half* __restrict__ dst, const int* __restrict__ offsets,
                  const int* __restrict__ counts, int E) {
  constexpr int K = H, R = 2 * I;
  constexpr int MT = I / TILE_M;  // tiles per expert: 4
  constexpr int NSTEP = K / KC;   // 16
  extern __shared__ unsigned char dyn_raw[];
  unsigned char* dyn = reinterpret_cast<unsigned char*>(((uintptr_t)dyn_raw + 1023) & ~(uintptr_t)1023);
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* aring = dyn + CTL_BYTES;
  unsigned char* bring = aring + NSA * A_STAGE;
  unsigned char* tabs = bring + NSB * B_STAGE;
  int* base = reinterpret_cast<int*>(tabs + NTAB * TAB_SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_wait();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSA; ++s) mbar_init(&ctl.afull[s], 1), mbar_init(&ctl.aempty[s], 1);
    for (int s = 0; s < NSB; ++s) mbar_init(&ctl.bfull[s], PREP_WARPS), mbar_init(&ctl.bempty[s], 1);
    for (int s = 0; s < 2; ++s) mbar_init(&ctl.accfull[s], 1), mbar_init(&ctl.accfree[s], PREP_WARPS);
    for (int s = 0; s < NTAB; ++s) mbar_init(&ctl.tabfull[s], 1), mbar_init(&ctl.tabempty[s], PREP_WARPS);
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&ctl.tmem_base, TMEM_COLS);
  if (warp == 0) {  // items per expert, exclusive prefix in base[]
    int carry = 0;
    for (int s0 = 0; s0 < E; s0 += 32) {
      const int s = s0 + lane;
      const int cnt = s < E ? __ldg(counts + s) : 0;
      const int items = ((cnt + NT - 1) / NT) * MT;
      int incl = items;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (s < E) base[s] = carry + incl - items;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) base[E] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  const int total_items = base[E];

  struct Item {
    int e, mt, n0;
  };
  auto decode = [&](int item) {
    int lo = 0, hi = E;  // the last expert whose range starts at or before the item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (base[mid] <= item) lo = mid;
      else hi = mid;
    }
    Item it;
    it.e = lo;
    const int local = item - base[lo];
    it.mt = local % MT;
    it.n0 = (local / MT) * NT;
    return it;
  };
  // table slot: token rows [NT] | (unused) [NT] | c of accumulator 0, 1 [NT each] | scales of block row 0, 1 [MAX_KB each] | nt
  auto tab_row = [&](unsigned n) { return reinterpret_cast<int*>(tabs + (n % NTAB) * TAB_SLOT); };
  auto tab_c = [&](unsigned n, int w) { return reinterpret_cast<float*>(tab_row(n) + 2 * NT) + w * NT; };
  auto tab_s = [&](unsigned n, int w) { return reinterpret_cast<float*>(tab_row(n) + 4 * NT) + w * MAX_KB; };
  auto tab_nt = [&](unsigned n) { return tab_row(n) + 4 * NT + 2 * MAX_KB; };
  // the 128-row box of the expert's rows (= block row of the scale array) behind accumulator w of tile mt
  auto block_row = [&](int mt, int w) { return w * (I / TILE_M) + mt; };

  bool dead = false;   // a wait ran out once: stop waiting (the error word is set; results are void)
  unsigned st_no = 0;  // steps so far (every role counts alike)
  unsigned it_no = 0;  // items so far

  if (warp == LOAD_WARP) {
    // ================= loader: lane 0 requests the step's two weight boxes =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item it = decode(item);
      for (int step = 0; step < NSTEP; ++step, ++st_no) {
        const int s = st_no % NSA;
        if (st_no >= NSA && !dead) dead = !mbar_wait_hot(&ctl.aempty[s], ((st_no / NSA) - 1) & 1, DRB_ERR_EMPTY_WAIT);
        if (lane == 0) {
          unsigned char* dstp = aring + (size_t)s * A_STAGE;
          mbar_expect_tx(&ctl.afull[s], A_STAGE);
#pragma unroll
          for (int w = 0; w < NACC; ++w)
            tma_load_2d(dstp + w * A_BYTES, &tm, step * KC, it.e * R + block_row(it.mt, w) * TILE_M, &ctl.afull[s]);
        }
        __syncwarp();
      }
    }
    // Tail: the MMA warp's completion arrivals for the last stages are in flight until they land; the block must not
    // end (and hand its shared memory to a successor) before they have.
    for (unsigned k = st_no > NSA ? st_no - NSA : 0; k < st_no; ++k)
      if (!dead) dead = !mbar_wait(&ctl.aempty[k % NSA], (k / NSA) & 1, DRB_ERR_EMPTY_WAIT);
  } else if (warp == MMA_WARP) {
    // ================= MMA warp: lane 0 issues both accumulators' MMAs =================
    // One issuing thread per block, as in every tcgen05 kernel this library has run for long: a variant with one issuing
    // warp per accumulator raised rare launch failures (about one in 150 back-to-back calls) that reading did not explain.
    const uint32_t idesc = instr_desc_e4m3(NCOL);
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const int a = it_no & 1;
      if (it_no >= 2 && !dead) dead = !mbar_wait_hot(&ctl.accfree[a], ((it_no >> 1) - 1) & 1, DRB_ERR_TMEM);
      for (int step = 0; step < NSTEP; ++step, ++st_no) {
        const int sa = st_no % NSA, sb = st_no % NSB;
        if (!dead) dead = !mbar_wait_hot(&ctl.bfull[sb], (st_no / NSB) & 1, DRB_ERR_TMEM);
        if (!dead) dead = !mbar_wait_hot(&ctl.afull[sa], (st_no / NSA) & 1, DRB_ERR_TMEM);
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int w = 0; w < NACC; ++w) {
            const uint32_t acc = tmem + (uint32_t)((a * NACC + w) * NCOL);
            const uint64_t ad = smem_desc(aring + (size_t)sa * A_STAGE + w * A_BYTES);
            const uint64_t bd = smem_desc(bring + (size_t)sb * B_STAGE + w * TERMS * BT_BYTES);  // 48 rows: the three terms
#pragma unroll
            for (int k32 = 0; k32 < KC / 32; ++k32) mma_e4m3(acc, ad + 2 * k32, bd + 2 * k32, idesc, step > 0 || k32 > 0);
          }
          mma_commit(&ctl.aempty[sa]);
          mma_commit(&ctl.bempty[sb]);
          if (step == NSTEP - 1) mma_commit(&ctl.accfull[a]);
        }
        __syncwarp();
      }
    }
  } else if (warp == TABLE_WARP) {
    // ================= table warp: one item ahead: token rows, the two block rows' scales, every token's c =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (it_no >= NTAB && !dead) dead = !mbar_wait(&ctl.tabempty[it_no % NTAB], ((it_no / NTAB) - 1) & 1, DRB_ERR_EMPTY_WAIT);
      const int cnt = __ldg(counts + it.e), off = __ldg(offsets + it.e);
      const int nt = min(NT, cnt - it.n0);
      const int row = off + it.n0 + (lane < nt ? lane : 0);
      const float rm = lane < nt ? __ldg(rmax + row) : 0.f;
#pragma unroll
      for (int w = 0; w < NACC; ++w) {
        const float sv = lane < NSTEP ? __ldg(S + ((size_t)it.e * (R / TILE_M) + block_row(it.mt, w)) * NSTEP + lane) : 0.f;
        if (lane < NSTEP) tab_s(it_no, w)[lane] = sv;
        const float c = rm * warp_max(fabsf(sv)) * (1.f / 256.f);
        if (lane < NT) tab_c(it_no, w)[lane] = (c > 1.0e-30f && c <= 3.0e38f) ? c : 1.f;
      }
      if (lane < NT) tab_row(it_no)[lane] = row;
      if (lane == 0) tab_nt(it_no)[0] = nt;
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tabfull[it_no % NTAB]);
    }
  } else {
    // ================= prep warps: the token tiles B', and the epilogue =================
    const int pt = threadIdx.x;         // 0 .. 127
    const int t = pt >> 3, c = pt & 7;  // token and 16-input piece of the chunk this thread prepares
    const int r = warp * 32 + lane;     // tile row in the epilogue (warp = tensor-memory lane quarter)
    const uint32_t b_off = swz_off(t, c);
    // An item's epilogue: accumulators [128 units (lanes), nt tokens (columns)] -> SiLU(gate) * up -> act.
    auto epilogue = [&](const Item& pit, unsigned pno) {
      const int nt = tab_nt(pno)[0];
      const int* rows = tab_row(pno);
      const int a = pno & 1;
      if (!dead) dead = !mbar_wait_hot(&ctl.accfull[a], (pno >> 1) & 1, DRB_ERR_TMEM);
      tc_fence_after();
      float g[NT], u[NT];
#pragma unroll
      for (int j = 0; j < TERMS; ++j) {  // the three terms' column groups add up
        uint32_t v0[16], v1[16];
        tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)((a * NACC) * NCOL + j * NT), v0);
        tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)((a * NACC + 1) * NCOL + j * NT), v1);
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          g[i] = j == 0 ? __uint_as_float(v0[i]) : g[i] + __uint_as_float(v0[i]);
          u[i] = j == 0 ? __uint_as_float(v1[i]) : u[i] + __uint_as_float(v1[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.accfree[a]);
      const float* c0 = tab_c(pno, 0);
      const float* c1 = tab_c(pno, 1);
#pragma unroll
      for (int i = 0; i < NT; ++i)
        if (i < nt) {
          dst[(size_t)rows[i] * I + pit.mt * TILE_M + r] = f2h_sat(silu_f(g[i] * c0[i]) * (u[i] * c1[i]));
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tabempty[pno % NTAB]);
    };
    Item pend_it = {};
    unsigned pend_no = 0;
    bool pending = false;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (!dead) dead = !mbar_wait(&ctl.tabfull[it_no % NTAB], (it_no / NTAB) & 1, DRB_ERR_FULL_WAIT);
      const int nt = tab_nt(it_no)[0];
      const bool live = t < nt;
      const uint4* rowp = reinterpret_cast<const uint4*>(src + (size_t)tab_row(it_no)[t] * K + 16 * c);
      float inv_c[NACC];
#pragma unroll
      for (int w = 0; w < NACC; ++w) inv_c[w] = 1.f / tab_c(it_no, w)[t];
      uint4 xl = make_uint4(0u, 0u, 0u, 0u), xh = xl;
      if (live) xl = __ldg(rowp), xh = __ldg(rowp + 1);
      for (int step = 0; step < NSTEP; ++step, ++st_no) {
        const int sb = st_no % NSB;
        const uint32_t xs[8] = {xl.x, xl.y, xl.z, xl.w, xh.x, xh.y, xh.z, xh.w};
        if (live && step + 1 < NSTEP) xl = __ldg(rowp + (step + 1) * (KC / 8)), xh = __ldg(rowp + (step + 1) * (KC / 8) + 1);
        // the MMAs that read this stage NSB steps ago must have completed
        if (st_no >= NSB && !dead) dead = !mbar_wait_hot(&ctl.bempty[sb], ((st_no / NSB) - 1) & 1, DRB_ERR_TMEM);
        unsigned char* bt = bring + (size_t)sb * B_STAGE;
#pragma unroll
        for (int w = 0; w < NACC; ++w) {
          const float f = tab_s(it_no, w)[step] * inv_c[w];
          uint32_t o[TERMS][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pa[TERMS], pb[TERMS];
            split3(__uint_as_float(xs[2 * q] << 16) * f, __uint_as_float(xs[2 * q] & 0xffff0000u) * f, pa);
            split3(__uint_as_float(xs[2 * q + 1] << 16) * f, __uint_as_float(xs[2 * q + 1] & 0xffff0000u) * f, pb);
#pragma unroll
            for (int j = 0; j < TERMS; ++j) o[j][q] = pa[j] | (pb[j] << 16);
          }
          if (live) {
#pragma unroll
            for (int j = 0; j < TERMS; ++j)
              *reinterpret_cast<uint4*>(bt + (w * TERMS + j) * BT_BYTES + b_off) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
          }
        }
        fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.bfull[sb]);
        if (step == 0 && pending) {  // the previous item's accumulators, while this item's first MMAs run
          epilogue(pend_it, pend_no);
          pending = false;
        }
      }
      pend_it = it, pend_no = it_no, pending = true;
    }
    if (pending) epilogue(pend_it, pend_no);
    for (unsigned k = st_no > NSB ? st_no - NSB : 0; k < st_no; ++k)  // tail: see the loader's
      if (!dead) dead = !mbar_wait(&ctl.bempty[k % NSB], (k / NSB) & 1, DRB_ERR_TMEM);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- the down projection ------------------------------------------------------------------------------------------
// K is only four chunks here and a tile is 64 KB, so a work item of one tile would spend more on its token tile, its
// table entry and its hand-overs than on its weights. Instead the chunk's scale stays out of the token operand:
// B'[t][k] = act[t][k] / c_t serves EVERY tile of the expert, each chunk of a tile has an accumulator of its own (four of
// 48 columns, used as a ring: the epilogue drains chunk kb of one tile while the MMAs of the next chunks run), and the
// epilogue forms c_t * sum_kb s[tile][kb] * acc_kb. A work item is (expert, group of up to 16 tokens, four consecutive
// tiles): B' is prepared once per item (24 KB, two items' worth resident) by two operand warps that run an item ahead,
// four epilogue warps do nothing but drain accumulators (the MMA warp waits for a free accumulator otherwise), the
// table warp reads each token row once per item and runs two items ahead, and the weights stream through a ring of
// 16 KB boxes, one per chunk.
namespace down {

constexpr int EPI_WARPS = 4, OPER_WARPS = 2;
constexpr int OPER_WARP0 = EPI_WARPS, MMA_W = EPI_WARPS + OPER_WARPS, LOAD_W = MMA_W + 1, TABLE_W = MMA_W + 2;
constexpr int THREADS = (TABLE_W + 1) * 32;  // 288
constexpr int NKB = I / KC;                 // 4 chunks = 4 accumulators per tile
constexpr int TPI = 4;                      // tiles per item
constexpr int QPE = H / TILE_M / TPI;       // items per expert and token group: 4
constexpr int NSA = 3;                      // weight boxes in flight
constexpr int NTAB = 3;                     // table slots: the table warp runs two items ahead
constexpr int BI_BYTES = NKB * TERMS * BT_BYTES;  // one item's token operand: 24 KB
constexpr int TAB_SLOT = (NT + NT + TPI * NKB) * 4 + 16;  // token rows | c | scales [tile][chunk] | nt
constexpr size_t SMEM = 1024 + CTL_BYTES + (size_t)NSA * A_BYTES + 2 * BI_BYTES + NTAB * TAB_SLOT + BASE_BYTES;
constexpr int TMEM_COLS = 256;              // four accumulators of 48 columns = 192, rounded up
static_assert(NKB * NCOL <= TMEM_COLS, "tensor memory");
static_assert(SMEM <= 113 * 1024, "two blocks per multiprocessor");

struct Ctl {
  uint64_t afull[NSA], aempty[NSA];    // a weight box landed / the MMAs that read it completed
  uint64_t bfull[2][NKB], bempty[2];   // a chunk of an item's token operand written (one arrival per operand warp) / the item's MMAs completed
  uint64_t accfull[NKB], accfree[NKB]; // a chunk's accumulator complete / drained (one arrival per epilogue warp)
  uint64_t tabfull[NTAB], tabempty[NTAB];  // an item's table written / read for the last time (operand and epilogue warps)
  uint32_t tmem_base;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block");

// tm: d_w as a tensor map over [E * H rows, I bytes]. S: f32 [E, H / 128, I / 128]. src: act fp16 [slots, I]. dst: y f32 [slots, H].
__global__ void __launch_bounds__(THREADS, 2)
    k_down_fp8(const __grid_constant__ CUtensorMap tm, const float* __restrict__ S, const __half* __restrict__ src,
               float* __restrict__ dst, const int* __restrict__ offsets, const int* __restrict__ counts, int E) {
  extern __shared__ unsigned char dyn_raw[];
  unsigned char* dyn = reinterpret_cast<unsigned char*>(((uintptr_t)dyn_raw + 1023) & ~(uintptr_t)1023);
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* aring = dyn + CTL_BYTES;
  unsigned char* bbuf = aring + NSA * A_BYTES;
  unsigned char* tabs = bbuf + 2 * BI_BYTES;
  int* base = reinterpret_cast<int*>(tabs + NTAB * TAB_SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_wait();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSA; ++s) mbar_init(&ctl.afull[s], 1), mbar_init(&ctl.aempty[s], 1);
    for (int s = 0; s < 2; ++s) {
      for (int kb = 0; kb < NKB; ++kb) mbar_init(&ctl.bfull[s][kb], OPER_WARPS);
      mbar_init(&ctl.bempty[s], 1);
    }
    for (int kb = 0; kb < NKB; ++kb) mbar_init(&ctl.accfull[kb], 1), mbar_init(&ctl.accfree[kb], EPI_WARPS);
    for (int s = 0; s < NTAB; ++s) mbar_init(&ctl.tabfull[s], 1), mbar_init(&ctl.tabempty[s], EPI_WARPS + OPER_WARPS);
    mbar_fence_init();
  }
  if (warp == MMA_W) tmem_alloc(&ctl.tmem_base, TMEM_COLS);
  if (warp == 0) {  // items per expert, exclusive prefix in base[]
    int carry = 0;
    for (int s0 = 0; s0 < E; s0 += 32) {
      const int s = s0 + lane;
      const int cnt = s < E ? __ldg(counts + s) : 0;
      const int items = ((cnt + NT - 1) / NT) * QPE;
      int incl = items;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (s < E) base[s] = carry + incl - items;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) base[E] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  const int total_items = base[E];

  struct Item {
    int e, q, n0;
  };
  auto decode = [&](int item) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (base[mid] <= item) lo = mid;
      else hi = mid;
    }
    Item it;
    it.e = lo;
    const int local = item - base[lo];
    it.q = local % QPE;
    it.n0 = (local / QPE) * NT;
    return it;
  };
  auto tab_row = [&](unsigned n) { return reinterpret_cast<int*>(tabs + (n % NTAB) * TAB_SLOT); };
  auto tab_c = [&](unsigned n) { return reinterpret_cast<float*>(tab_row(n) + NT); };
  auto tab_s = [&](unsigned n) { return reinterpret_cast<float*>(tab_row(n) + 2 * NT); };
  auto tab_nt = [&](unsigned n) { return tab_row(n) + 2 * NT + TPI * NKB; };

  bool dead = false;
  unsigned it_no = 0;  // items so far
  unsigned ch_no = 0;  // weight boxes so far (loader and MMA warp count alike)

  if (warp == LOAD_W) {
    // ================= loader: lane 0 requests a weight box per chunk =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item it = decode(item);
      for (int i = 0; i < TPI; ++i)
        for (int kb = 0; kb < NKB; ++kb, ++ch_no) {
          const int s = ch_no % NSA;
          if (ch_no >= NSA && !dead) dead = !mbar_wait_hot(&ctl.aempty[s], ((ch_no / NSA) - 1) & 1, DRB_ERR_EMPTY_WAIT);
          if (lane == 0) {
            mbar_expect_tx(&ctl.afull[s], A_BYTES);
            tma_load_2d(aring + (size_t)s * A_BYTES, &tm, kb * KC, it.e * H + (it.q * TPI + i) * TILE_M, &ctl.afull[s]);
          }
          __syncwarp();
        }
    }
    // Tail: the block must not end before the completion arrivals for its last boxes have landed.
    for (unsigned k = ch_no > NSA ? ch_no - NSA : 0; k < ch_no; ++k)
      if (!dead) dead = !mbar_wait(&ctl.aempty[k % NSA], (k / NSA) & 1, DRB_ERR_EMPTY_WAIT);
  } else if (warp == MMA_W) {
    // ================= MMA warp: lane 0 issues; chunk kb of a tile goes into accumulator kb =================
    const uint32_t idesc = instr_desc_e4m3(NCOL);
    unsigned tl_no = 0;  // tiles so far
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const int ip = it_no & 1;
      for (int i = 0; i < TPI; ++i, ++tl_no) {
        for (int kb = 0; kb < NKB; ++kb, ++ch_no) {
          const int sa = ch_no % NSA;
          if (tl_no >= 1 && !dead) dead = !mbar_wait_hot(&ctl.accfree[kb], (tl_no - 1) & 1, DRB_ERR_TMEM);
          if (i == 0 && !dead) dead = !mbar_wait_hot(&ctl.bfull[ip][kb], (it_no >> 1) & 1, DRB_ERR_TMEM);
          if (!dead) dead = !mbar_wait_hot(&ctl.afull[sa], (ch_no / NSA) & 1, DRB_ERR_TMEM);
          tc_fence_after();
          if (lane == 0) {
            const uint32_t acc = tmem + (uint32_t)(kb * NCOL);
            const uint64_t ad = smem_desc(aring + (size_t)sa * A_BYTES);
            const uint64_t bd = smem_desc(bbuf + (size_t)ip * BI_BYTES + kb * TERMS * BT_BYTES);  // 48 rows: the three terms
#pragma unroll
            for (int k32 = 0; k32 < KC / 32; ++k32) mma_e4m3(acc, ad + 2 * k32, bd + 2 * k32, idesc, k32 > 0);
            mma_commit(&ctl.aempty[sa]);
            if (i == TPI - 1 && kb == NKB - 1) mma_commit(&ctl.bempty[ip]);
            mma_commit(&ctl.accfull[kb]);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == TABLE_W) {
    // ================= table warp: two items ahead =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (it_no >= NTAB && !dead) dead = !mbar_wait(&ctl.tabempty[it_no % NTAB], ((it_no / NTAB) - 1) & 1, DRB_ERR_EMPTY_WAIT);
      const int cnt = __ldg(counts + it.e), off = __ldg(offsets + it.e);
      const int nt = min(NT, cnt - it.n0);
      if (lane < TPI * NKB) tab_s(it_no)[lane] = __ldg(S + ((size_t)it.e * (H / TILE_M) + it.q * TPI) * NKB + lane);
      // every token row's largest magnitude, eight rows per round trip (fp16 with the sign cleared orders like an integer)
      constexpr int TB = 8;
      for (int t0 = 0; t0 < NT; t0 += TB) {
        uint4 v[TB][2];
#pragma unroll
        for (int u = 0; u < TB; ++u) {
          const int row = off + it.n0 + (t0 + u < nt ? t0 + u : 0);
          const uint4* p = reinterpret_cast<const uint4*>(src + (size_t)row * I);
          v[u][0] = __ldcg(p + lane), v[u][1] = __ldcg(p + 32 + lane);
        }
#pragma unroll
        for (int u = 0; u < TB; ++u) {
          const uint32_t wv[8] = {v[u][0].x, v[u][0].y, v[u][0].z, v[u][0].w, v[u][1].x, v[u][1].y, v[u][1].z, v[u][1].w};
          uint32_t m = 0u;
#pragma unroll
          for (int q = 0; q < 8; ++q) m = max(m, max(wv[q] & 0x7fffu, (wv[q] >> 16) & 0x7fffu));
          m = __reduce_max_sync(0xffffffffu, m);
          if (lane == 0) {
            const float c = __half2float(__ushort_as_half((unsigned short)m)) * (1.f / 256.f);
            tab_row(it_no)[t0 + u] = off + it.n0 + (t0 + u < nt ? t0 + u : 0);
            tab_c(it_no)[t0 + u] = (t0 + u < nt && c > 1.0e-30f && c <= 3.0e38f) ? c : 1.f;
          }
        }
      }
      if (lane == 0) tab_nt(it_no)[0] = nt;
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tabfull[it_no % NTAB]);
    }
  } else if (warp >= OPER_WARP0) {
    // ================= operand warps: an item's token operand, three E4M3 terms of act / c_t =================
    const int po = threadIdx.x - OPER_WARP0 * 32;  // 0 .. 63
    const int c = po & 7, t0 = po >> 3;            // 16-input piece; tokens t0 and t0 + 8
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const int ip = it_no & 1;
      if (!dead) dead = !mbar_wait(&ctl.tabfull[it_no % NTAB], (it_no / NTAB) & 1, DRB_ERR_FULL_WAIT);
      // the MMAs of the item before last read this buffer
      if (it_no >= 2 && !dead) dead = !mbar_wait(&ctl.bempty[ip], ((it_no >> 1) - 1) & 1, DRB_ERR_TMEM);
      const int nt = tab_nt(it_no)[0];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int t = t0 + half * (NT / 2);
        const bool live = t < nt;
        const float inv_c = 1.f / tab_c(it_no)[t];
        const uint4* rowp = reinterpret_cast<const uint4*>(src + (size_t)tab_row(it_no)[t] * I + 16 * c);
        const uint32_t b_off = swz_off(t, c);
        uint4 xl[NKB], xh[NKB];
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          xl[kb] = xh[kb] = make_uint4(0u, 0u, 0u, 0u);
          if (live) xl[kb] = __ldcg(rowp + kb * (KC / 8)), xh[kb] = __ldcg(rowp + kb * (KC / 8) + 1);
        }
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          const uint32_t xs[8] = {xl[kb].x, xl[kb].y, xl[kb].z, xl[kb].w, xh[kb].x, xh[kb].y, xh[kb].z, xh[kb].w};
          uint32_t o[TERMS][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pa[TERMS], pb[TERMS];
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&xs[2 * q]));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&xs[2 * q + 1]));
            split3(fa.x * inv_c, fa.y * inv_c, pa);
            split3(fb.x * inv_c, fb.y * inv_c, pb);
#pragma unroll
            for (int j = 0; j < TERMS; ++j) o[j][q] = pa[j] | (pb[j] << 16);
          }
          if (live) {
            unsigned char* bt = bbuf + (size_t)ip * BI_BYTES + kb * TERMS * BT_BYTES;
#pragma unroll
            for (int j = 0; j < TERMS; ++j) *reinterpret_cast<uint4*>(bt + j * BT_BYTES + b_off) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
          }
        }
      }
      fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) mbar_arrive(&ctl.bfull[ip][kb]);
        mbar_arrive(&ctl.tabempty[it_no % NTAB]);
      }
    }
    for (unsigned n = it_no > 2 ? it_no - 2 : 0; n < it_no; ++n)  // tail: see the loader's
      if (!dead) dead = !mbar_wait(&ctl.bempty[n & 1], (n >> 1) & 1, DRB_ERR_TMEM);
  } else {
    // ================= epilogue warps: drain every tile's four accumulators =================
    const int r = warp * 32 + lane;  // tile row (warp = tensor-memory lane quarter)
    unsigned tl_no = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (!dead) dead = !mbar_wait(&ctl.tabfull[it_no % NTAB], (it_no / NTAB) & 1, DRB_ERR_FULL_WAIT);
      const int nt = tab_nt(it_no)[0];
      const int* rows = tab_row(it_no);
      const float* cs = tab_c(it_no);
      for (int i = 0; i < TPI; ++i, ++tl_no) {
        const float* sc = tab_s(it_no) + i * NKB;
        const int mt = it.q * TPI + i;
        float sum[NT];
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          if (!dead) dead = !mbar_wait_hot(&ctl.accfull[kb], tl_no & 1, DRB_ERR_TMEM);
          tc_fence_after();
          const float s = sc[kb];
#pragma unroll
          for (int j = 0; j < TERMS; ++j) {  // the three terms' column groups add up
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(kb * NCOL + j * NT), v);
#pragma unroll
            for (int q = 0; q < NT; ++q) sum[q] = (kb == 0 && j == 0) ? s * __uint_as_float(v[q]) : fmaf(s, __uint_as_float(v[q]), sum[q]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.accfree[kb]);
        }
#pragma unroll
        for (int q = 0; q < NT; ++q)
          if (q < nt) dst[(size_t)rows[q] * H + mt * TILE_M + r] = sum[q] * cs[q];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tabempty[it_no % NTAB]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_W) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace down

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(k_gate_up_fp8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(down::k_down_fp8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)down::SMEM)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_gate_up_fp8)) != cudaSuccess) return e;
  return drb_carveout(down::k_down_fp8);
}

}  // namespace pf8
