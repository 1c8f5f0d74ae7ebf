// Expert-grouped prefill on the 5th-generation tensor cores: dr_moe_prefill as two grouped GEMMs
// whose int4 weights are dequantised straight into tcgen05 operand tiles.
//
//   gate/up:  for expert e with its cnt tokens  D[128, cnt] = W_tile[128, 2048] . X_e[cnt, 2048]^T
//             (the tile interleaves 64 gate rows with their 64 up rows), epilogue silu(g) * u -> act
//   down:     D[128, cnt] = Wd_tile[128, 512] . act_e[cnt, 512]^T -> y
//
// "Swap-AB": the weight rows are the MMA's M = 128 dimension and the tokens its N dimension
// (16 .. 64, rounded up to 16; larger groups take several accumulators), because most experts see a handful of
// tokens: with Zipf routing of 300 rows the median group is 4 tokens. Accumulators live in tensor memory
// (64 columns of fp32).
//
// One persistent block per multiprocessor walks the (expert, 128-row tile) items. Per 64-wide
// K chunk (= one int4 scale group) its 256 threads
//   * dequantise 128 x 64 nibbles to fp16 (w = q*scale + min, single rounding) and store them in the
//     K-major 128-byte-swizzled layout the MMA reads (A operand),
//   * convert the tokens' 64 activations to fp16 in the same element order (B operand),
// and one thread issues four tcgen05.mma.kind::f16 (K = 16 each). Four chunk stages let the
// dequantisation of chunk k+1 overlap the MMAs of chunk k; tcgen05.commit on an mbarrier frees a stage.
// fp16 operands (not bf16): bf16-dequantised weights miss the 1e-3 output tolerance (1.65e-3), fp16
// measures 1.8e-4.
//
// Every wait is bounded (common.cuh); tensor memory is allocated once per block and always freed.
// Replaces kernels/drama.cu:799-968 of the reference (k_moe_pf_gate_up, k_moe_pf_down).
#pragma once

#include "common.cuh"

namespace pfmma {

constexpr int H = 2048, I = 512;
constexpr int PRODUCER_WARPS = 8;                   // two blocks per multiprocessor
constexpr int BLOCKS_PER_SM = 16 / PRODUCER_WARPS;
constexpr int PRODUCERS = PRODUCER_WARPS * 32;
constexpr int THREADS = PRODUCERS + 32;             // + the MMA-issuing warp
constexpr int TILE_M = 128;
constexpr int KC = 64;                              // K chunk = one swizzle atom of fp16 = one int4 scale group
constexpr int MAX_N = 64;                           // tokens per accumulator (one work item)
constexpr int NG = 4;                               // token groups enumerated per expert; the last one loops on
constexpr int A_BYTES = TILE_M * KC * 2;            // 16 KB
constexpr int B_BYTES = MAX_N * KC * 2;             // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 24 KB; four stages: two blocks fit a multiprocessor
constexpr int STAGES = 4;
constexpr int CTL_BYTES = 1024;
constexpr size_t SMEM_BYTES = CTL_BYTES + 1024 /* alignment slack */ + (size_t)STAGES * STAGE_BYTES;  // 98 KB
constexpr int TMEM_COLS = MAX_N;
constexpr int BPT = MAX_N * 8 / PRODUCERS;             // 16-byte B chunks per thread and K chunk
constexpr int SPLIT = PRODUCERS / TILE_M;              // threads per tile row: 2
constexpr int NST = 8 / SPLIT;                         // 16-byte operand chunks a thread writes per K chunk: 4
static_assert(BPT >= 1 && SPLIT == 2, "operand mapping");

struct Ctl {
  uint64_t full[STAGES];   // a stage has been filled (one arrival per producer warp)
  uint64_t empty[STAGES];  // a stage's MMAs have completed
  uint64_t done;           // all MMAs of the current accumulator have completed
  uint64_t tfree;          // the accumulator has been read out (one arrival per epilogue warp)
  uint32_t tmem_base;
};

// ---- tcgen05 wrappers ------------------------------------------------------------------------

DRB_DEV void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
DRB_DEV void tmem_dealloc(uint32_t base, uint32_t cols) {  // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
DRB_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DRB_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DRB_DEV void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
DRB_DEV uint64_t smem_desc(const void* p) {
  const uint64_t addr = (uint64_t)(smem_u32(p) >> 4) & 0x3FFFull;
  return addr | (1ull << 16) /* leading offset: unused with swizzle */ | (64ull << 32) /* 1024 B >> 4 */ |
         (1ull << 46) /* descriptor version */ | (2ull << 61) /* SWIZZLE_128B */;
}

// Instruction descriptor for kind::f16: fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n.
DRB_DEV uint32_t instr_desc(int n) {
  return (1u << 4) /* D = f32 */ | (0u << 7) /* A = f16 */ | (0u << 10) /* B = f16 */ | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

DRB_DEV void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}

// Arrives on `bar` once every MMA issued so far by this thread has completed.
DRB_DEV void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive fp32 columns of this warp's 32 lanes.
DRB_DEV void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Byte offset of 16-byte chunk c (0..7) of row r inside a K-major 128-byte-swizzled tile.
DRB_DEV uint32_t swz_off(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

// Eight nibbles of one word -> eight fp16 weights q*s + m, in element order (0,4,1,5,2,6,3,7).
// 0x6400 | q is the half 1024 + q; subtracting 1024 is exact, the fused multiply-add rounds once.
DRB_DEV uint4 dequant8(uint32_t w, __half2 s2, __half2 m2) {
  const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
  uint32_t t[4];
  t[0] = lop3_and_or(w, 0x000F000Fu, 0x64006400u);
  t[1] = lop3_and_or(w >> 4, 0x000F000Fu, 0x64006400u);
  t[2] = lop3_and_or(w >> 8, 0x000F000Fu, 0x64006400u);
  t[3] = lop3_and_or(w >> 12, 0x000F000Fu, 0x64006400u);
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 q = __hsub2(*reinterpret_cast<__half2*>(&t[i]), k1024);
    const __half2 r = __hfma2(q, s2, m2);
    op[i] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return o;
}

// Sixteen E4M3 weights (k ascending) times one block scale -> sixteen fp16 in k order. s2 holds the scale, already
// multiplied by the row block's power of two (see k_grouped), in both halves; the product rounds once.
DRB_DEV void dequant16_fp8(const uint4& v, __half2 s2, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t a, b;
    asm("{.reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t;}" : "=r"(a) : "r"(w[i] & 0xffffu));
    asm("{.reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t;}" : "=r"(b) : "r"(w[i] >> 16));
    const __half2 pa = __hmul2(*reinterpret_cast<const __half2*>(&a), s2), pb = __hmul2(*reinterpret_cast<const __half2*>(&b), s2);
    o[2 * i] = *reinterpret_cast<const uint32_t*>(&pa), o[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&pb);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// 2^-floor(log2(s)) for a positive finite s: s times it lies in [1, 2).
DRB_DEV float pow2_normaliser(float s) {
  const int e = (int)((__float_as_uint(s) >> 23) & 0xffu);  // biased exponent (0 for zero / subnormal: treated as 2^-126)
  return __uint_as_float((uint32_t)(254 - (e ? e : 1)) << 23);
}

// The power of two that brings a block row's LARGEST scale into [1, 2): every scale of the row times it is at most 2,
// so an E4M3 weight (at most 448) times its normalised scale stays inside fp16 however far the row's scales are apart.
DRB_DEV float block_row_normaliser(const float* scales, int n) {
  float m = 0.f;
  for (int i = 0; i < n; ++i) m = fmaxf(m, fabsf(__ldg(scales + i)));
  return pow2_normaliser(m);
}

// Two floats -> packed fp16 (lo, hi), round to nearest, clamped to the largest finite fp16: the operands of the
// tensor-core path are fp16, whose range ends at 65504 where bf16 and fp32 carry on. An outlier beyond it then
// degrades (it is clamped) instead of turning a token's whole output row into NaN through an infinity.
DRB_DEV uint32_t f2h2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
DRB_DEV __half f2h_sat(float v) {
  unsigned short h;
  asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
  return __ushort_as_half(h);
}

// Eight bf16 activations (k ascending) -> fp16 in k order.
DRB_DEV uint4 bf16x8_to_f16_nat(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) op[i] = f2h2_sat(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  return o;
}

// Sixteen int8 weights (k ascending) times one fp16 scale -> sixteen fp16 in k order. 0x6400 | (b ^ 0x80) is the
// half 1024 + 128 + b; subtracting 1152 is exact, the product rounds once.
DRB_DEV void dequant16_i8(const uint4& v, __half2 s2, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  const __half2 k1152 = __half2half2(__ushort_as_half((unsigned short)0x6480));
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t u = w[i] ^ 0x80808080u;
    const uint32_t a = prmt(u, 0x64646464u, 0x4140u), b = prmt(u, 0x64646464u, 0x4342u);
    const __half2 pa = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&a), k1152), s2);
    const __half2 pb = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&b), k1152), s2);
    o[2 * i] = *reinterpret_cast<const uint32_t*>(&pa), o[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&pb);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// Eight bf16 activations (k ascending) -> fp16 in the same (0,4,1,5,2,6,3,7) order.
DRB_DEV uint4 bf16x8_to_f16_perm(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};  // (0,1) (2,3) (4,5) (6,7)
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) f[2 * i] = __uint_as_float(w[i] << 16), f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) op[i] = f2h2_sat(f[i], f[i + 4]);
  return o;
}

// Eight fp16 (k ascending) -> the (0,4,1,5,2,6,3,7) order.
DRB_DEV uint4 f16x8_perm(const uint4& v) {
  uint4 o;
  o.x = prmt(v.x, v.z, 0x5410u);  // (0, 4)
  o.y = prmt(v.x, v.z, 0x7632u);  // (1, 5)
  o.z = prmt(v.y, v.w, 0x5410u);  // (2, 6)
  o.w = prmt(v.y, v.w, 0x7632u);  // (3, 7)
  return o;
}


// The int8 shared expert, run by the same launch as one more "expert" that owns every row (SH = true). Its work
// items (one per 64-token group and 128-row tile) come first: they are the largest.
struct SharedExpert {
  const int8_t* q;  // gate/up: [2I, H]; down: [H, I]
  const __half* s;  // one scale per 128 inputs: [rows of q, K / 128]
  const void* src;  // gate/up: the normalised rows, bf16 [rows, H], in row order; down: fp16 [rows, I]
  void* dst;        // gate/up: fp16 [rows, I]; down: f32 [rows, H]
  int rows;
};

// GEMM = 0: gate/up (+ SwiGLU, fp16 out);  GEMM = 1: down (fp32 out).
// FMT = 0: int4 experts: Q [E, R, K/2] nibbles, SM [E, R, K/64] (scale, min);  R = 2I, K = H for gate/up;  R = H, K = I for down.
// FMT = 1: block-FP8 experts: Q [E, R, K] E4M3 bytes, SM = f32 scales [E, R/128, K/128]. A row block's scales are
//   brought into fp16 range by the power of two that normalises the block row's largest scale (the weights times the
//   scaled scale round once to fp16); the epilogue multiplies the row's result by the inverse power, exactly.
//   src: gate/up: xp bf16 [slots, H] (or, with row_of, the unpermuted rows [rows, H] and row_of[slot]; fp16 rows when
//        src_f16 is set: three more significant bits than bf16, which the 1e-3 bar against fp32 rows needs);  down: act fp16 [slots, I]
//   dst: gate/up: act fp16 [slots, I]; down: y f32 [slots, H]
// Warps 0-7 convert operands into the stage ring and run the epilogue; warp 8 issues the MMAs. They meet only
// on mbarriers: full[s] (8 warp arrivals), empty[s] and done (tcgen05.commit), tfree (accumulator drained).
template <int GEMM, int FMT = 0, bool SH = false>
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM)
    k_grouped(const uint8_t* __restrict__ Q, const void* __restrict__ SMv, const void* __restrict__ src, void* __restrict__ dst,
              const int* __restrict__ offsets, const int* __restrict__ counts, int E, SharedExpert sh,
              const int* __restrict__ row_of, int src_f16, const int* __restrict__ dst_row_of) {
  const __half2* SM = static_cast<const __half2*>(SMv);  // FMT 0
  const float* SF = static_cast<const float*>(SMv);      // FMT 1
  constexpr int K = GEMM == 0 ? H : I;
  constexpr int R = GEMM == 0 ? 2 * I : H;
  constexpr int MT = R / TILE_M;  // tiles per expert: 8 / 16
  constexpr int NKC = K / KC;     // 32 / 8
  constexpr int ESZ = 2;          // both activation sources are 16-bit
  extern __shared__ unsigned char dyn_raw[];
  unsigned char* dyn = reinterpret_cast<unsigned char*>(((uintptr_t)dyn_raw + 1023) & ~(uintptr_t)1023);
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  unsigned char* stages = dyn + CTL_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_wait();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl.empty[s], 1);
      mbar_init(&ctl.full[s], PRODUCER_WARPS);
    }
    mbar_init(&ctl.done, 1);
    mbar_init(&ctl.tfree, PRODUCER_WARPS);
    mbar_fence_init();
  }
  if (warp == PRODUCER_WARPS) tmem_alloc(&ctl.tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;

  bool dead = false;      // a wait ran out once: stop waiting (the error word is set; results are void)
  unsigned chunk_no = 0;  // chunks so far: selects stage and mbarrier phase (same sequence in every warp)
  unsigned acc_no = 0;    // accumulators so far: phase of `done` and `tfree`

  // Work items, walked in the same order by every warp: the shared expert's (token group, tile) pairs, then the routed
  // experts' (expert, token group, tile) triples; the last enumerated group of a routed expert also takes whatever
  // lies beyond NG * MAX_N tokens.
  const int sh_items = SH ? ((sh.rows + MAX_N - 1) / MAX_N) * MT : 0;
  const int total_items = sh_items + E * NG * MT;
  struct Item {
    bool valid, shared, single;
    int e, mt, cnt, nfirst;
  };
  auto decode = [&](int item) {
    Item it;
    it.shared = SH && item < sh_items;
    if (it.shared) {
      it.mt = item % MT, it.nfirst = (item / MT) * MAX_N, it.cnt = sh.rows, it.e = 0, it.single = true, it.valid = true;
    } else {
      const int i2 = item - sh_items;
      const int g = (i2 / MT) % NG;
      it.mt = i2 % MT, it.e = i2 / (MT * NG), it.cnt = counts[it.e], it.nfirst = g * MAX_N, it.single = g != NG - 1;
      it.valid = it.nfirst < it.cnt;
    }
    return it;
  };

  if (warp == PRODUCER_WARPS) {
    // ================= MMA warp =================
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item it = decode(item);
      if (!it.valid) continue;
      for (int n0 = it.nfirst; n0 < it.cnt; n0 += MAX_N) {
        if (n0 > it.nfirst && it.single) break;
        const int N = (min(MAX_N, it.cnt - n0) + 15) & ~15;
        const uint32_t idesc = instr_desc(N);
        // the previous accumulator must have been read out
        if (acc_no > 0 && !dead) dead = !mbar_wait(&ctl.tfree, (acc_no - 1) & 1, DRB_ERR_TMEM);
        tc_fence_after();
        for (int kc = 0; kc < NKC; ++kc, ++chunk_no) {
          const int s = chunk_no % STAGES;
          if (!dead) dead = !mbar_wait(&ctl.full[s], (chunk_no / STAGES) & 1, DRB_ERR_TMEM);
          tc_fence_after();
          if (lane == 0) {
            unsigned char* As = stages + (size_t)s * STAGE_BYTES;
            const uint64_t ad = smem_desc(As), bd = smem_desc(As + A_BYTES);
#pragma unroll
            for (int k16 = 0; k16 < KC / 16; ++k16) mma_f16(tmem, ad + 2 * k16, bd + 2 * k16, idesc, kc > 0 || k16 > 0);
            mma_commit(&ctl.empty[s]);
            if (kc == NKC - 1) mma_commit(&ctl.done);
          }
          __syncwarp();
        }
        ++acc_no;
      }
    }
  } else {
    // ================= producer / epilogue warps =================
    // This thread's share of the A tile: tile row t / 2, 32 of the chunk's 64 weights -> four 16-byte operand chunks.
    const int arow = threadIdx.x / SPLIT, ahalf = threadIdx.x % SPLIT;
    uint32_t a_off[NST];
#pragma unroll
    for (int j = 0; j < NST; ++j) a_off[j] = swz_off(arow, NST * ahalf + j);
    // Its share of the B tile: 16-byte chunk c of token n for idx = t + i * 256.
    uint32_t b_off[BPT];
#pragma unroll
    for (int i = 0; i < BPT; ++i) b_off[i] = A_BYTES + swz_off((threadIdx.x + i * PRODUCERS) >> 3, threadIdx.x & 7);
    const int q4 = warp & 3;       // tensor-memory lane quarter this warp may read
    const int r = q4 * 32 + lane;  // tile row in the epilogue
    constexpr int CB_R = FMT == 0 ? KC / 2 : KC;  // bytes of one K chunk of a routed weight row; this thread takes half of them
    constexpr int CB_S = KC;                      // the same of a shared-expert (int8) row
    constexpr int NL_R = CB_R / SPLIT / 16, NL_S = CB_S / SPLIT / 16;  // 16-byte pieces this thread loads per chunk: 1 or 2
    constexpr int NLX = SH ? (NL_S > NL_R ? NL_S : NL_R) : NL_R;
    static_assert(NL_R >= 1 && NL_S >= 1, "a thread loads whole 16-byte pieces");

    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item it = decode(item);
      if (!it.valid) continue;
      const bool shd = it.shared;
      const int mt = it.mt, e = it.e;
      const int off = shd ? 0 : offsets[e];
      // weight row of tile row r: gate/up interleaves gate j (even r) with up j (odd r)
      const int wrow = GEMM == 0 ? (arow & 1) * I + mt * (TILE_M / 2) + (arow >> 1) : mt * TILE_M + arow;
      const int cb = shd ? CB_S : CB_R;
      const uint8_t* qrow = shd ? reinterpret_cast<const uint8_t*>(sh.q) + (size_t)wrow * K + ahalf * (CB_S / SPLIT)
                                : Q + ((size_t)e * R + wrow) * (FMT == 0 ? K / 2 : K) + ahalf * (CB_R / SPLIT);
      const __half2* smrow = SM + ((size_t)e * R + wrow) * (K / 64);
      const float* sfrow = SF + ((size_t)e * (R / 128) + (wrow >> 7)) * (K / 128);  // FMT 1: this row block's scales
      const __half* ssrow = sh.s + (size_t)wrow * (K / 128);                        // shared expert: this row's scales
      const float norm = (FMT == 1 && !shd) ? block_row_normaliser(sfrow, K / 128) : 1.f;
      const unsigned char* asrc = static_cast<const unsigned char*>(shd ? sh.src : src);
      void* adst = shd ? sh.dst : dst;
      const int nl = shd ? NL_S : NL_R;

      for (int n0 = it.nfirst; n0 < it.cnt; n0 += MAX_N) {
        if (n0 > it.nfirst && it.single) break;
        const int nt = min(MAX_N, it.cnt - n0);
        const int N = (nt + 15) & ~15;
        // activation rows of this thread's B chunks (nullptr beyond the group)
        const unsigned char* bsrc[BPT];
#pragma unroll
        for (int i = 0; i < BPT; ++i) {
          const int n = (threadIdx.x + i * PRODUCERS) >> 3;
          // row_of (gate/up of the routed experts only): slot -> row of src, so that no permuted copy of the rows is needed
          bsrc[i] = nullptr;
          if (n < nt) {
            const int slot = off + n0 + n;
            const int row = (GEMM == 0 && !shd && row_of) ? __ldg(row_of + slot) : slot;
            bsrc[i] = asrc + ((size_t)row * K) * ESZ + (threadIdx.x & 7) * 16;
          }
        }
        auto load_b = [&](int kc, int i) -> uint4 {
          if (!bsrc[i]) return make_uint4(0u, 0u, 0u, 0u);
          const uint4* p = reinterpret_cast<const uint4*>(bsrc[i] + (size_t)kc * KC * ESZ);
          return GEMM == 0 ? __ldg(p) : __ldcg(p);
        };
        // weights two chunks ahead, activations one chunk ahead, all in registers
        auto load_w = [&](int kc, int piece) -> uint4 {
          return __ldg(reinterpret_cast<const uint4*>(qrow + (size_t)kc * cb + 16 * piece));
        };
        uint4 q0[NLX], q1[NLX];
#pragma unroll
        for (int l = 0; l < NLX; ++l)
          if (l < nl) q0[l] = load_w(0, l), q1[l] = NKC > 1 ? load_w(1, l) : q0[l];
        __half2 sm0 = (FMT == 0 && !shd) ? __ldg(smrow) : __half2();
        __half2 sm1 = (FMT == 0 && !shd) ? (NKC > 1 ? __ldg(smrow + 1) : sm0) : __half2();
        uint4 bn[BPT];
#pragma unroll
        for (int i = 0; i < BPT; ++i) bn[i] = load_b(0, i);
        for (int kc = 0; kc < NKC; ++kc, ++chunk_no) {
          const int s = chunk_no % STAGES;
          unsigned char* st = stages + (size_t)s * STAGE_BYTES;
          uint4 qv[NLX];
#pragma unroll
          for (int l = 0; l < NLX; ++l) qv[l] = q0[l], q0[l] = q1[l];
          const __half2 smv = sm0;
          sm0 = sm1;
          if (kc + 2 < NKC) {
#pragma unroll
            for (int l = 0; l < NLX; ++l)
              if (l < nl) q1[l] = load_w(kc + 2, l);
            if (FMT == 0 && !shd) sm1 = __ldg(smrow + kc + 2);
          }
          uint4 bv[BPT];
#pragma unroll
          for (int i = 0; i < BPT; ++i) bv[i] = bn[i];
          if (kc + 1 < NKC) {
#pragma unroll
            for (int i = 0; i < BPT; ++i) bn[i] = load_b(kc + 1, i);
          }
          // the MMAs that read this stage STAGES chunks ago must have completed
          if (chunk_no >= STAGES && !dead) dead = !mbar_wait(&ctl.empty[s], ((chunk_no / STAGES) - 1) & 1, DRB_ERR_TMEM);
          bool natural;  // element order of the operand chunks: k ascending, or (0,4,1,5,2,6,3,7) within each eight
          if (SH && shd) {
            natural = true;
            const __half2 s2 = __half2half2(__ldg(ssrow + (kc >> 1)));  // one scale per 128 inputs = two chunks
#pragma unroll
            for (int l = 0; l < NL_S; ++l) {
              uint4 o0, o1;
              dequant16_i8(qv[l], s2, o0, o1);
              *reinterpret_cast<uint4*>(st + a_off[2 * l]) = o0, *reinterpret_cast<uint4*>(st + a_off[2 * l + 1]) = o1;
            }
          } else if (FMT == 0) {
            natural = false;
            const __half2 s2 = __half2half2(__low2half(smv)), m2 = __half2half2(__high2half(smv));
#pragma unroll
            for (int l = 0; l < NL_R; ++l) {
              const uint32_t w[4] = {qv[l].x, qv[l].y, qv[l].z, qv[l].w};
#pragma unroll
              for (int j = 0; j < NST / NL_R; ++j) *reinterpret_cast<uint4*>(st + a_off[l * (NST / NL_R) + j]) = dequant8(w[j], s2, m2);
            }
          } else {
            natural = true;
            const __half2 s2 = __float2half2_rn(__ldg(sfrow + (kc >> 1)) * norm);  // one scale per 128 inputs = two chunks
#pragma unroll
            for (int l = 0; l < NL_R; ++l) {
              uint4 o0, o1;
              dequant16_fp8(qv[l], s2, o0, o1);
              *reinterpret_cast<uint4*>(st + a_off[2 * l]) = o0, *reinterpret_cast<uint4*>(st + a_off[2 * l + 1]) = o1;
            }
          }
#pragma unroll
          for (int i = 0; i < BPT; ++i)
            if (bsrc[i]) {
              uint4 o;
              const bool from_bf16 = GEMM == 0 && !src_f16;  // the gate/up rows arrive as bf16 (the reference's ABI) or as fp16
              if (!natural) o = from_bf16 ? bf16x8_to_f16_perm(bv[i]) : f16x8_perm(bv[i]);
              else o = from_bf16 ? bf16x8_to_f16_nat(bv[i]) : bv[i];
              *reinterpret_cast<uint4*>(st + b_off[i]) = o;
            }
          fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl.full[s]);
        }
        // ---- epilogue: accumulator [128 tile rows (lanes), N tokens (columns)]
        if (!dead) dead = !mbar_wait(&ctl.done, acc_no & 1, DRB_ERR_TMEM);
        ++acc_no;
        tc_fence_after();
        // FMT 1: undo the power of two that normalised the scales of this tile row's 128-row block
        float unnorm = 1.f;
        if (FMT == 1 && !shd) {
          const int erow = GEMM == 0 ? (r & 1) * I + mt * (TILE_M / 2) + (r >> 1) : mt * TILE_M + r;
          unnorm = 1.f / block_row_normaliser(SF + ((size_t)e * (R / 128) + (erow >> 7)) * (K / 128), K / 128);
        }
        for (int c0 = (warp >> 2) * 16; c0 < N; c0 += 4 * PRODUCER_WARPS) {  // each set of four warps takes every (PRODUCER_WARPS / 4)-th 16-column group
          uint32_t v[16];
          tmem_ld16(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0, v);
          if (FMT == 1) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * unnorm);
          }
          if (GEMM == 0) {
            __half* act = static_cast<__half*>(adst);
            const int j = mt * (TILE_M / 2) + (r >> 1);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float mine = __uint_as_float(v[i]);
              const float other = __shfl_xor_sync(0xffffffffu, mine, 1);  // even lane: gate, odd lane: up
              if ((lane & 1) == 0 && c0 + i < nt) act[(size_t)(off + n0 + c0 + i) * I + j] = f2h_sat(silu_f(mine) * other);
            }
          } else {
            float* y = static_cast<float*>(adst);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c0 + i < nt) {
                // dst_row_of (down projection of the routed experts only): slot -> row of y, so that the results land where
                // their consumer wants them (an expert-parallel rank: in the order the rows arrived)
                const int slot = off + n0 + c0 + i;
                const int row = (!shd && dst_row_of) ? __ldg(dst_row_of + slot) : slot;
                y[(size_t)row * H + mt * TILE_M + r] = __uint_as_float(v[i]);
              }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.tfree);  // this warp has drained its part of the accumulator
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == PRODUCER_WARPS) tmem_dealloc(tmem, TMEM_COLS);
}

template <typename Kn>
static cudaError_t configure_one(Kn kernel) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  return e != cudaSuccess ? e : drb_carveout(kernel);
}

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = configure_one(k_grouped<0, 0, false>)) != cudaSuccess) return e;
  if ((e = configure_one(k_grouped<1, 0, false>)) != cudaSuccess) return e;
  if ((e = configure_one(k_grouped<0, 0, true>)) != cudaSuccess) return e;
  if ((e = configure_one(k_grouped<1, 0, true>)) != cudaSuccess) return e;
  if ((e = configure_one(k_grouped<0, 1, false>)) != cudaSuccess) return e;
  return configure_one(k_grouped<1, 1, false>);
}

}  // namespace pfmma
