// The grouped prefill GEMMs of drb_moe_prefill_block: pfmma::k_grouped's arithmetic (int4 / int8 weights dequantised
// to fp16 with the group scale applied, tcgen05.mma.kind::f16, fp32 accumulators in tensor memory) with every load
// taken off the warps that dequantise.
//
// pfmma::k_grouped spends about six thread-instructions per weight, of which two are the dequantisation; the rest
// are the weight loads and their address arithmetic, the register queues that hide their latency, the token tile's
// loads and conversion, and the swizzle offsets. Here
//   loader warp   one tiled TMA request per raw stage: 128 tile rows x 128 bytes (256 int4 or 128 int8 inputs of
//                 every row) with the 128-byte swizzle; a gate/up tile arrives with gate row j and up row j
//                 interleaved, which a 4-D view of the weight tensor expresses (row byte, gate|up, unit, expert)
//   token warp    the tokens' fp16 rows -> B tiles by asynchronous 16-byte copies (cp.async), straight into the
//                 swizzled layout, as far ahead as the stage ring allows
//   table warp    one item ahead, the item's token rows (a chain of dependent global loads)
//   8 convert warps  per 64-input chunk and thread: one 16-byte piece out of shared memory, dequantise, four (int4)
//                 or two x two (int8) 16-byte stores; the row's scales come 16 bytes at a time, one raw stage ahead
//   MMA warp      four K = 16 instructions per chunk into one of two accumulators; tcgen05.commit frees the stage
// and the convert warps drain an item's accumulator (SwiGLU / store) while the MMAs of the next item run into the
// other accumulator. Roles meet only on mbarriers; every wait is bounded (common.cuh).
//
// Work items: (shared expert or expert, group of up to 64 tokens, 128-row tile), enumerated from the device-side
// counts by a prefix sum each block computes for itself, the shared expert's items first.
// Replaces kernels/drama.cu:799-968 of the reference (k_moe_pf_gate_up, k_moe_pf_down) together with the cuBLAS
// shared expert of src/engine.rs:351-355, 560-562.
#pragma once

#include <type_traits>

#include <cuda.h>  // CUtensorMap and the encode function's type only: the entry point is resolved at run time

#include "common.cuh"
#include "moe_prefill_mma.cuh"

namespace pft {

using pfmma::dequant16_i8;
using pfmma::f2h_sat;
using pfmma::fence_async_smem;
using pfmma::instr_desc;
using pfmma::mma_commit;
using pfmma::mma_f16;
using pfmma::smem_desc;
using pfmma::swz_off;
using pfmma::tc_fence_after;
using pfmma::tc_fence_before;
using pfmma::tmem_alloc;
using pfmma::tmem_dealloc;
using pfmma::tmem_ld16;

constexpr int H = 2048, I = 512;
constexpr int CONVERT_WARPS = 8, CONVERTERS = CONVERT_WARPS * 32;
constexpr int MMA_WARP = CONVERT_WARPS, LOAD_WARP = CONVERT_WARPS + 1, TABLE_WARP = CONVERT_WARPS + 2, TOKEN_WARP = CONVERT_WARPS + 3;
constexpr int THREADS = CONVERTERS + 128;  // 12 warps at 80 registers: two blocks per multiprocessor
constexpr int TILE_M = 128;
constexpr int KC = 64;                     // K chunk = one swizzle row of fp16 = one int4 scale group
constexpr int NT = 32;                     // tokens per work item = accumulator columns
constexpr int NACC = 2;
constexpr int TMEM_COLS = NACC * NT;
constexpr int ROW_BYTES = 128;
constexpr int RAW_BYTES = TILE_M * ROW_BYTES;  // 16 KB: 256 int4 or 128 int8 inputs of the tile's 128 rows
constexpr int NRAW = 2;
constexpr int A_BYTES = TILE_M * KC * 2;       // 16 KB
constexpr int B_BYTES = NT * KC * 2;           // 4 KB
constexpr int NST = 3;                         // A tiles in flight
constexpr int NBT = 6;                         // B tiles in flight: a token tile comes from L2 and takes longer than an A tile's conversion
constexpr int MAX_ITEM_SETS = 256 + 1;         // experts + the shared expert
constexpr int CTL_BYTES = 1024;
constexpr int TAB_SLOT = 2 * NT * 4 + 16;      // per item: operand rows, result rows, token count
constexpr int NTAB = 2;
constexpr int BASE_BYTES = ((MAX_ITEM_SETS + 1) * 4 + 127) / 128 * 128;
constexpr size_t SMEM_BYTES = 1024 /* alignment slack */ + CTL_BYTES + NRAW * RAW_BYTES + NST * A_BYTES + NBT * B_BYTES + NTAB * TAB_SLOT + BASE_BYTES;
static_assert(SMEM_BYTES <= 113 * 1024, "two blocks per multiprocessor");
constexpr int BPL = NT * 8 / 32;               // 16-byte B pieces per lane of the token warp and chunk

struct Ctl {
  uint64_t rawfull[NRAW];   // the TMA request of a raw stage has landed (transaction count)
  uint64_t rawempty[NRAW];  // it has been converted (one arrival per convert warp)
  uint64_t full[NST];       // an A tile has been written (one arrival per convert warp)
  uint64_t empty[NST];      // the MMAs that read the A tile have completed (tcgen05.commit)
  uint64_t bfull[NBT];      // a B tile has landed (the token warp)
  uint64_t bempty[NBT];     // the MMAs that read the B tile have completed (tcgen05.commit)
  uint64_t accfull[NACC];   // an item's accumulator is complete (tcgen05.commit)
  uint64_t accfree[NACC];   // it has been drained (one arrival per convert warp)
  uint64_t tabfull[NTAB];   // an item's tables have been written (the table warp)
  uint64_t tabempty[NTAB];  // the item is finished (one arrival per convert warp)
  uint32_t tmem_base;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block");

// Tiled TMA loads into shared memory, completing on an mbarrier. The tensor maps live in kernel parameter space.
DRB_DEV void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
               : "memory");
}
DRB_DEV void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// Eight nibbles of one word -> eight fp16 weights q*s + m in k order. A nibble in bits 0..3 of a 16-bit half, or-ed
// into 0x6400, is the half 1024 + q; a nibble in bits 4..7, or-ed into 0x5400, is the half 64 + q (the unit in the last
// place of 64 is 1/16, sixteen of them per step of the nibble): one shift serves the upper byte of both halves.
// Subtracting the offset is exact, the fused multiply-add rounds once.
DRB_DEV uint4 dequant8_nat(uint32_t w, __half2 s2, __half2 m2) {
  const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
  const __half2 k64 = __half2half2(__ushort_as_half((unsigned short)0x5400));
  const uint32_t w8 = w >> 8;
  uint32_t t[4];  // (k0, k4), (k1, k5), (k2, k6), (k3, k7)
  t[0] = lop3_and_or(w, 0x000F000Fu, 0x64006400u);
  t[1] = lop3_and_or(w, 0x00F000F0u, 0x54005400u);
  t[2] = lop3_and_or(w8, 0x000F000Fu, 0x64006400u);
  t[3] = lop3_and_or(w8, 0x00F000F0u, 0x54005400u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 r = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t[i]), (i & 1) ? k64 : k1024), s2, m2);
    t[i] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return make_uint4(prmt(t[0], t[1], 0x5410u), prmt(t[2], t[3], 0x5410u), prmt(t[0], t[1], 0x7632u), prmt(t[2], t[3], 0x7632u));
}

// GEMM = 0: gate/up + SwiGLU -> act fp16 [., I];  GEMM = 1: down -> y f32 [., H].
//   tm_q / SM: the routed experts, int4 through a tensor map + (scale, min) [E, R, K/64];  tm_sh / shs: the shared
//   expert, int8 through a tensor map + scale [R, K/128];  R = 2I, K = H for gate/up;  R = H, K = I for down.
//   src / sh_src: fp16 rows [., K] in k order for the routed experts / the shared expert. gate/up: both are the
//   normalised rows, a routed token's row is row_of[slot] (or slot), the shared expert's token n is row n;  down:
//   the two act arrays, row slot / row n.
//   dst / sh_dst: gate/up: act fp16 [., I], row slot / row n;  down: f32 [., H], row dst_row_of[slot] (or slot) / row n.
//   peer_y (down, routed results only; or NULL): device array of every rank's result buffer. dst_row_of[slot] = s * cap + j
//   then names the token's source rank s and its slot j there, and the row is stored straight into rank s's buffer
//   at row rank * cap + j over NVLink: the GEMM's epilogue is the second half of the expert-parallel exchange.
template <int GEMM>
__global__ void __launch_bounds__(THREADS, 2)
    k_grouped_tma(const __grid_constant__ CUtensorMap tm_q, const __half2* __restrict__ SM, const __grid_constant__ CUtensorMap tm_sh,
                  const __half* __restrict__ shs, const __half* __restrict__ src, const __half* __restrict__ sh_src,
                  void* __restrict__ dst, void* __restrict__ sh_dst, const int* __restrict__ offsets, const int* __restrict__ counts, int E, int rows_sh,
                  const int* __restrict__ row_of, const int* __restrict__ dst_row_of, float* const* __restrict__ peer_y, int peer_cap,
                  int peer_rank) {
  constexpr int K = GEMM == 0 ? H : I;
  constexpr int R = GEMM == 0 ? 2 * I : H;
  constexpr int MT = R / TILE_M;  // tiles per expert: 8 / 16
  constexpr int NKC = K / KC;     // chunks along K: 32 / 8
  extern __shared__ unsigned char dyn_raw[];
  unsigned char* dyn = reinterpret_cast<unsigned char*>(((uintptr_t)dyn_raw + 1023) & ~(uintptr_t)1023);
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* raw = dyn + CTL_BYTES;
  unsigned char* stages = raw + NRAW * RAW_BYTES;
  unsigned char* bring = stages + NST * A_BYTES;
  unsigned char* tabs = bring + NBT * B_BYTES;
  int* base = reinterpret_cast<int*>(tabs + NTAB * TAB_SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_wait();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NRAW; ++s) mbar_init(&ctl.rawfull[s], 1), mbar_init(&ctl.rawempty[s], CONVERT_WARPS);
    for (int s = 0; s < NST; ++s) mbar_init(&ctl.full[s], CONVERT_WARPS), mbar_init(&ctl.empty[s], 1);
    for (int s = 0; s < NBT; ++s) mbar_init(&ctl.bfull[s], 1), mbar_init(&ctl.bempty[s], 1);
    for (int s = 0; s < NACC; ++s) mbar_init(&ctl.accfull[s], 1), mbar_init(&ctl.accfree[s], CONVERT_WARPS);
    for (int s = 0; s < NTAB; ++s) mbar_init(&ctl.tabfull[s], 1), mbar_init(&ctl.tabempty[s], CONVERT_WARPS);
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&ctl.tmem_base, TMEM_COLS);
  // Items per set (set 0: the shared expert, set 1 + e: expert e), exclusive prefix in base[]: warp 0 scans.
  const int n_sets = E + 1;
  if (warp == 0) {
    int carry = 0;
    for (int s0 = 0; s0 < n_sets; s0 += 32) {
      const int s = s0 + lane;
      int cnt = 0;
      if (s < n_sets) cnt = s == 0 ? rows_sh : __ldg(counts + s - 1);
      const int items = ((cnt + NT - 1) / NT) * MT;
      int incl = items;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (s < n_sets) base[s] = carry + incl - items;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) base[n_sets] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  const int total_items = base[n_sets];

  struct Item {
    bool shared;
    int e, mt, n0;
  };
  auto decode = [&](int item) {
    int lo = 0, hi = n_sets;  // the last set whose range starts at or before the item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (base[mid] <= item) lo = mid;
      else hi = mid;
    }
    Item it;
    it.shared = lo == 0;
    it.e = lo - 1;
    const int local = item - base[lo];
    it.mt = local % MT;
    it.n0 = (local / MT) * NT;
    return it;
  };
  // weight row of tile row r: a gate/up tile interleaves gate j (even r) with up j (odd r)
  auto weight_row = [&](int mt, int r) { return GEMM == 0 ? (r & 1) * I + mt * (TILE_M / 2) + (r >> 1) : mt * TILE_M + r; };
  auto tab_row = [&](unsigned n) { return reinterpret_cast<int*>(tabs + (n % NTAB) * TAB_SLOT); };  // [NT] operand rows
  auto tab_dst = [&](unsigned n) { return tab_row(n) + NT; };                                       // [NT] result rows
  auto tab_nt = [&](unsigned n) { return tab_dst(n) + NT; };                                        // token count

  bool dead = false;    // a wait ran out once: stop waiting (the error word is set; results are void)
  unsigned raw_no = 0;  // raw stages so far (loader, convert warps)
  unsigned ch_no = 0;   // chunks = stages so far (convert, MMA, token warps)
  unsigned it_no = 0;   // items so far

  if (warp == LOAD_WARP) {
    // ================= loader: lane 0 requests one box per raw stage =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item it = decode(item);
      const int nraw = (it.shared ? K : K / 2) / ROW_BYTES;
      for (int rs = 0; rs < nraw; ++rs, ++raw_no) {
        const int s = raw_no % NRAW;
        if (raw_no >= NRAW && !dead) dead = !mbar_wait(&ctl.rawempty[s], ((raw_no / NRAW) - 1) & 1, DRB_ERR_EMPTY_WAIT);
        if (lane == 0) {
          unsigned char* dstp = raw + (size_t)s * RAW_BYTES;
          mbar_expect_tx(&ctl.rawfull[s], RAW_BYTES);
          const CUtensorMap* map = it.shared ? &tm_sh : &tm_q;
          if (GEMM == 0) tma_load_4d(dstp, map, rs * ROW_BYTES, 0, it.mt * (TILE_M / 2), it.shared ? 0 : it.e, &ctl.rawfull[s]);
          else tma_load_2d(dstp, map, rs * ROW_BYTES, (it.shared ? 0 : it.e * R) + it.mt * TILE_M, &ctl.rawfull[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == MMA_WARP) {
    // ================= MMA warp =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      if (!dead) dead = !mbar_wait(&ctl.tabfull[it_no % NTAB], (it_no / NTAB) & 1, DRB_ERR_FULL_WAIT);
      const int nt = tab_nt(it_no)[0];
      const uint32_t idesc = instr_desc((nt + 15) & ~15);
      const int a = it_no % NACC;
      if (it_no >= NACC && !dead) dead = !mbar_wait(&ctl.accfree[a], ((it_no / NACC) - 1) & 1, DRB_ERR_TMEM);
      for (int kc = 0; kc < NKC; ++kc, ++ch_no) {
        const int s = ch_no % NST, sb = ch_no % NBT;
        if (!dead) dead = !mbar_wait(&ctl.bfull[sb], (ch_no / NBT) & 1, DRB_ERR_TMEM);
        if (!dead) dead = !mbar_wait(&ctl.full[s], (ch_no / NST) & 1, DRB_ERR_TMEM);
        tc_fence_after();
        if (lane == 0) {
          const uint64_t ad = smem_desc(stages + (size_t)s * A_BYTES), bd = smem_desc(bring + (size_t)sb * B_BYTES);
#pragma unroll
          for (int k16 = 0; k16 < KC / 16; ++k16) mma_f16(tmem + (uint32_t)(a * NT), ad + 2 * k16, bd + 2 * k16, idesc, kc > 0 || k16 > 0);
          mma_commit(&ctl.empty[s]);
          mma_commit(&ctl.bempty[sb]);
          if (kc == NKC - 1) mma_commit(&ctl.accfull[a]);
        }
        __syncwarp();
      }
    }
  } else if (warp == TOKEN_WARP) {
    // ================= token warp: the tokens' fp16 rows -> B tiles =================
    unsigned b_done = 0;     // B tiles announced so far (ch_no counts the requested ones)
    auto announce = [&]() {  // the oldest requested tile has landed
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.bfull[b_done % NBT]);
      ++b_done;
    };
    // Announces requested tiles, oldest first, each as soon as it has landed, until at most `keep` are still under way
    // (cp.async.wait_group takes its count as an immediate: one instance per possible count).
    auto settle = [&](unsigned requested, unsigned keep) {
      static_assert(NBT == 6, "one step per possible count");
      auto step = [&](auto n) {
        if (requested - b_done > (unsigned)decltype(n)::value && (unsigned)decltype(n)::value >= keep) {
          asm volatile("cp.async.wait_group %0;" ::"n"(decltype(n)::value) : "memory");
          announce();
        }
      };
      step(std::integral_constant<int, 5>{});
      step(std::integral_constant<int, 4>{});
      step(std::integral_constant<int, 3>{});
      step(std::integral_constant<int, 2>{});
      step(std::integral_constant<int, 1>{});
      step(std::integral_constant<int, 0>{});
    };
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (!dead) dead = !mbar_wait(&ctl.tabfull[it_no % NTAB], (it_no / NTAB) & 1, DRB_ERR_FULL_WAIT);
      const int nt = tab_nt(it_no)[0];
      const int* trow = tab_row(it_no);
      const unsigned char* rows = reinterpret_cast<const unsigned char*>(it.shared ? sh_src : src);
      // this lane's pieces: 16-byte piece c of token t's 128-byte row segment, t = lane / 8 + 4 i
      const unsigned char* bsrc[BPL];
      uint32_t bdst[BPL];
#pragma unroll
      for (int i = 0; i < BPL; ++i) {
        const int t = (lane >> 3) + 4 * i, c = lane & 7;
        bsrc[i] = nullptr, bdst[i] = 0;
        if (t < nt) {
          bsrc[i] = rows + (size_t)trow[t] * K * 2 + 16 * c;
          bdst[i] = swz_off(t, c);
        }
      }
      for (int kc = 0; kc < NKC; ++kc, ++ch_no) {
        const int s = ch_no % NBT;
        if (ch_no >= NBT && !dead) {
          // Before a wait that may block, announce everything that is under way: a tile must not be held back by
          // the request for a later one.
          if (!mbar_try_wait(&ctl.bempty[s], ((ch_no / NBT) - 1) & 1)) {
            settle(ch_no, 0);
            dead = !mbar_wait(&ctl.bempty[s], ((ch_no / NBT) - 1) & 1, DRB_ERR_EMPTY_WAIT);
          }
        }
        const uint32_t tile = smem_u32(bring + (size_t)s * B_BYTES);
#pragma unroll
        for (int i = 0; i < BPL; ++i)
          if (bsrc[i]) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tile + bdst[i]), "l"(bsrc[i] + (size_t)kc * KC * 2) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        settle(ch_no + 1, 2);  // two tiles stay under way (about an L2 round trip of requests); older ones are announced
      }
    }
    settle(ch_no, 0);
  } else if (warp == TABLE_WARP) {
    // ================= table warp: the tokens of every item, one item ahead =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      if (it_no >= NTAB && !dead) dead = !mbar_wait(&ctl.tabempty[it_no % NTAB], ((it_no / NTAB) - 1) & 1, DRB_ERR_EMPTY_WAIT);
      const int cnt = it.shared ? rows_sh : __ldg(counts + it.e);
      const int nt = min(NT, cnt - it.n0);
      const int off = it.shared ? 0 : __ldg(offsets + it.e);
#pragma unroll
      for (int i = 0; i < NT / 32; ++i) {
        const int t = lane + 32 * i;
        int row = 0, drow = 0;
        if (t < nt) {
          if (it.shared) {
            row = drow = it.n0 + t;
          } else {
            const int slot = off + it.n0 + t;
            row = (GEMM == 0 && row_of) ? __ldg(row_of + slot) : slot;
            drow = (GEMM == 1 && dst_row_of) ? __ldg(dst_row_of + slot) : slot;
          }
        }
        tab_row(it_no)[t] = row, tab_dst(it_no)[t] = drow;
      }
      if (lane == 0) tab_nt(it_no)[0] = nt;
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tabfull[it_no % NTAB]);
    }
  } else {
    // ================= convert warps: raw stage -> A tiles; then the item's epilogue =================
    const int ct = threadIdx.x;               // 0 .. 255
    const int arow = ct >> 1, ahalf = ct & 1;  // tile row and half of the chunk this thread converts
    const int q4 = warp & 3;                   // tensor-memory lane quarter this warp may read
    const int r = q4 * 32 + lane;              // tile row in the epilogue
    uint32_t a_off[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) a_off[j] = swz_off(arow, 4 * ahalf + j);
    // An item's epilogue: accumulator [128 tile rows (lanes), nt tokens (columns)] -> SwiGLU / store.
    auto epilogue = [&](const Item& pit, unsigned pno) {
      // ---- epilogue: accumulator [128 tile rows (lanes), nt tokens (columns)]
      if (!dead) dead = !mbar_wait(&ctl.tabfull[pno % NTAB], (pno / NTAB) & 1, DRB_ERR_FULL_WAIT);
      const int nt = tab_nt(pno)[0];
      const int* drow = tab_dst(pno);
      const int a = pno % NACC;
      if (!dead) dead = !mbar_wait(&ctl.accfull[a], (pno / NACC) & 1, DRB_ERR_TMEM);
      tc_fence_after();
      for (int c0 = (warp >> 2) * 16; c0 < nt; c0 += 32) {  // the two sets of four warps take one 16-column group each
        uint32_t v[16];
        tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * NT + c0), v);
        if (GEMM == 0) {
          __half* act = static_cast<__half*>(pit.shared ? sh_dst : dst);
          const int j = pit.mt * (TILE_M / 2) + (r >> 1);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float mine = __uint_as_float(v[i]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);  // even lane: gate, odd lane: up
            if ((lane & 1) == 0 && c0 + i < nt) act[(size_t)drow[c0 + i] * I + j] = f2h_sat(silu_f(mine) * other);
          }
        } else if (GEMM == 1 && peer_y && !pit.shared) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < nt) {
              const int q = drow[c0 + i], s = q / peer_cap;
              peer_y[s][((size_t)peer_rank * peer_cap + (q - s * peer_cap)) * H + pit.mt * TILE_M + r] = __uint_as_float(v[i]);
            }
          __threadfence_system();  // before the flag that a later kernel writes to the peers
        } else {
          float* y = static_cast<float*>(pit.shared ? sh_dst : dst);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < nt) y[(size_t)drow[c0 + i] * H + pit.mt * TILE_M + r] = __uint_as_float(v[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.accfree[a]), mbar_arrive(&ctl.tabempty[pno % NTAB]);
    };
    Item pend_it = {};
    unsigned pend_no = 0;
    bool pending = false;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it_no) {
      const Item it = decode(item);
      const bool shd = it.shared;
      const int wrow = weight_row(it.mt, arow);
      // this row's scales: int4: (scale, min) per chunk, 16 bytes = the four chunks of a raw stage; int8: one scale per
      // 128 inputs = per raw stage. Fetched one raw stage ahead.
      const uint4* smrow = reinterpret_cast<const uint4*>(SM + ((size_t)(shd ? 0 : it.e) * R + wrow) * NKC);
      const __half* ssrow = shs + (size_t)wrow * (K / 128);
      const int nraw = (shd ? K : K / 2) / ROW_BYTES;
      auto load_sc = [&](int rs) -> uint4 {
        if (rs >= nraw) return make_uint4(0u, 0u, 0u, 0u);
        if (shd) return make_uint4((uint32_t)__half_as_ushort(__ldg(ssrow + rs)), 0u, 0u, 0u);
        return __ldg(smrow + rs);
      };
      uint4 sc_next = load_sc(0);
      for (int rs = 0; rs < nraw; ++rs, ++raw_no) {
        const int sr = raw_no % NRAW;
        const uint4 sc = sc_next;
        sc_next = load_sc(rs + 1);
        if (!dead) dead = !mbar_wait(&ctl.rawfull[sr], (raw_no / NRAW) & 1, DRB_ERR_FULL_WAIT);
        const unsigned char* rawp = raw + (size_t)sr * RAW_BYTES;
        const int per_raw = shd ? 2 : 4;  // chunks in a raw stage
        const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll 4
        for (int cc = 0; cc < per_raw; ++cc, ++ch_no) {
          const int s = ch_no % NST;
          unsigned char* st = stages + (size_t)s * A_BYTES;
          uint4 x0, x1 = make_uint4(0u, 0u, 0u, 0u);
          if (shd) {
            x0 = *reinterpret_cast<const uint4*>(rawp + swz_off(arow, 4 * cc + 2 * ahalf));
            x1 = *reinterpret_cast<const uint4*>(rawp + swz_off(arow, 4 * cc + 2 * ahalf + 1));
          } else {
            x0 = *reinterpret_cast<const uint4*>(rawp + swz_off(arow, 2 * cc + ahalf));
          }
          // the MMAs that read this stage NST chunks ago must have completed
          if (ch_no >= NST && !dead) dead = !mbar_wait(&ctl.empty[s], ((ch_no / NST) - 1) & 1, DRB_ERR_TMEM);
          if (shd) {
            const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)(scw[0] & 0xffffu)));
            uint4 o0, o1, o2, o3;
            dequant16_i8(x0, s2, o0, o1);
            dequant16_i8(x1, s2, o2, o3);
            *reinterpret_cast<uint4*>(st + a_off[0]) = o0, *reinterpret_cast<uint4*>(st + a_off[1]) = o1;
            *reinterpret_cast<uint4*>(st + a_off[2]) = o2, *reinterpret_cast<uint4*>(st + a_off[3]) = o3;
          } else {
            const __half2 smv = *reinterpret_cast<const __half2*>(&scw[cc]);
            const __half2 s2 = __half2half2(__low2half(smv)), m2 = __half2half2(__high2half(smv));
            *reinterpret_cast<uint4*>(st + a_off[0]) = dequant8_nat(x0.x, s2, m2);
            *reinterpret_cast<uint4*>(st + a_off[1]) = dequant8_nat(x0.y, s2, m2);
            *reinterpret_cast<uint4*>(st + a_off[2]) = dequant8_nat(x0.z, s2, m2);
            *reinterpret_cast<uint4*>(st + a_off[3]) = dequant8_nat(x0.w, s2, m2);
          }
          fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.full[s]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.rawempty[sr]);
        if (rs == 0 && pending) {
          epilogue(pend_it, pend_no);
          pending = false;
        }
      }
      // The item's accumulator is drained after the first raw stage of the NEXT item has been converted: the MMAs of
      // its last chunks are still running when the conversion ends, and waiting for them here would idle the convert
      // warps once per item (measured: a third of a down item's time).
      pend_it = it, pend_no = it_no, pending = true;
    }
    if (pending) epilogue(pend_it, pend_no);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

// Tensor maps with the 128-byte swizzle the MMA's shared-memory descriptors expect, over byte matrices in the
// reference's layouts. cuTensorMapEncodeTiled is a driver entry point: it is looked up through the runtime once, so the
// library has no link-time dependency on the driver. Return 0 or -3.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static cudaError_t resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult status;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status);
  if (e != cudaSuccess) return e;
  if (status != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return cudaSuccess;
}

// Down projection: [rows, row_bytes] row-major, boxes of 128 rows x 128 bytes.
static int map_rows(CUtensorMap* map, const void* p, uint64_t rows, uint64_t row_bytes,
                    CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
  if (!g_encode) return -3;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {ROW_BYTES, TILE_M};
  const cuuint32_t estr[2] = {1, 1};
  return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? 0
             : -3;
}

// Gate/up: [experts][2 (gate | up)][units][row_bytes] seen as (row byte, gate|up, unit, expert); a box is 128 bytes of
// 64 units' gate row and up row, interleaved.
static int map_gate_up(CUtensorMap* map, const void* p, uint64_t experts, uint64_t units, uint64_t row_bytes) {
  if (!g_encode) return -3;
  const cuuint64_t dims[4] = {row_bytes, 2, units, experts};
  const cuuint64_t strides[3] = {units * row_bytes, row_bytes, 2 * units * row_bytes};
  const cuuint32_t box[4] = {ROW_BYTES, 2, TILE_M / 2, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? 0
             : -3;
}

template <typename Kn>
static cudaError_t configure_one(Kn kernel) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  return e != cudaSuccess ? e : drb_carveout(kernel);
}

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = resolve_encode()) != cudaSuccess) return e;
  if ((e = configure_one(k_grouped_tma<0>)) != cudaSuccess) return e;
  return configure_one(k_grouped_tma<1>);
}

}  // namespace pft
