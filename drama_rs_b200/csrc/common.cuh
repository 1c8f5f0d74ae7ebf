// Device-side building blocks shared by the sm_100a weight-streaming kernels.
//
//  * bulk asynchronous copies (TMA, `cp.async.bulk`) into shared memory that complete on an
//    mbarrier, with every wait bounded: a wait that runs out records a code in g_drb_error and
//    the kernel carries on to its end, so that a lost copy can never hang the device;
//  * programmatic dependent launch (`griddepcontrol`) so that a kernel's weight loads overlap
//    the tail of the kernel before it;
//  * in-register dequantisation of packed int4 / int8 to fp32 without the conversion unit, and
//    packed two-wide fp32 FMAs (`fma.rn.f32x2`).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DRB_DEV __device__ __forceinline__

// Error word written by kernels whose bounded waits ran out (0 = none). Read by drb_device_error().
// The library is one translation unit, so the definition lives here.
__device__ unsigned int g_drb_error = 0;

enum DrbError : unsigned int {
  DRB_OK = 0,
  DRB_ERR_FULL_WAIT = 1,   // a consumer gave up waiting for a bulk copy to land
  DRB_ERR_EMPTY_WAIT = 2,  // the producer gave up waiting for a free stage
  DRB_ERR_GRID_WAIT = 3,   // a grid-wide barrier did not complete
  DRB_ERR_TMEM = 4,        // tensor-memory allocation or MMA completion wait ran out
};

// ------------------------------------------------------------------------------------------
// small utilities

DRB_DEV float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

DRB_DEV float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

DRB_DEV float silu_f(float x) { return x / (1.f + expf(-x)); }
DRB_DEV float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

DRB_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Activation vectors are staged in shared memory as float4s at a swizzled index: thread t writes
// float4 t (coalesced global read), and a lane later reads the 4..8 consecutive float4s of its own
// k-slice. The XOR keeps both patterns free of bank conflicts for slices of 4, 8 or 16 floats... per lane.
DRB_DEV int swz4(int g) { return g ^ ((g >> 3) & 7); }

// ------------------------------------------------------------------------------------------
// programmatic dependent launch

// Blocks until the kernel this one depends on has completed and its writes are visible.
// A no-op when the kernel was launched without a programmatic dependency.
DRB_DEV void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream start its prologue.
DRB_DEV void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------------------------------
// mbarrier + bulk copies

DRB_DEV void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes barrier initialisation visible to the async proxy before the first copy names the barrier.
DRB_DEV void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

DRB_DEV void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

DRB_DEV void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

DRB_DEV bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: `limit` polls (by default about a second's worth), then the error word is set and the
// caller continues with whatever is in shared memory.
DRB_DEV bool mbar_wait(uint64_t* bar, unsigned parity, unsigned err_code, unsigned limit = 1u << 22) {
  for (unsigned it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(it > 4096 ? 256 : 32);
  }
  atomicMax(&g_drb_error, err_code);
  return false;
}

// The same for a wait on a ring's step-to-step path: no sleep between polls (a sleeping waiter adds its wake-up time
// to every hand-over of the ring), bounded all the same.
DRB_DEV bool mbar_wait_hot(uint64_t* bar, unsigned parity, unsigned err_code) {
  for (unsigned it = 0; it < (1u << 24); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  atomicMax(&g_drb_error, err_code);
  return false;
}

// Global -> shared bulk copy. dst, src 16-byte aligned; bytes a multiple of 16.
DRB_DEV void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Bulk L2 prefetch of [p, p + bytes): one instruction per region instead of one per 128-byte line.
// p 16-byte aligned; bytes a multiple of 16.
DRB_DEV void bulk_prefetch_l2(const void* p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Prefetches this block's share of [pf, pf + pf_bytes) into L2 (the next kernel's weights).
// Called by one thread per block. The region is cut into 16-byte aligned pieces of at most 64 KB.
DRB_DEV void prefetch_share(const char* pf, size_t pf_bytes, unsigned block, unsigned blocks) {
  if (!pf || pf_bytes == 0) return;
  const uintptr_t lo = ((uintptr_t)pf + 15) & ~(uintptr_t)15;
  const uintptr_t hi = ((uintptr_t)pf + pf_bytes) & ~(uintptr_t)15;
  if (hi <= lo) return;
  const size_t total = hi - lo;
  const size_t per = (((total + blocks - 1) / blocks) + 15) & ~(size_t)15;
  size_t b0 = (size_t)block * per;
  const size_t b1 = b0 + per < total ? b0 + per : total;
  while (b0 < b1) {
    const size_t n = b1 - b0 < 65536 ? b1 - b0 : 65536;
    bulk_prefetch_l2((const char*)lo + b0, (unsigned)n);
    b0 += n;
  }
}

// ------------------------------------------------------------------------------------------
// packed fp32 arithmetic: two FMAs per issued instruction

struct f2 {
  float x, y;
};

DRB_DEV unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

DRB_DEV void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// acc += a * b, lane-wise on two packed floats.
DRB_DEV unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long acc) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(acc));
  return r;
}

DRB_DEV unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

DRB_DEV uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

DRB_DEV uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// ------------------------------------------------------------------------------------------
// int4: eight nibbles of one 32-bit word against eight activations.
//
// Nibble q (0..15) is placed in mantissa bits 19..22 of 0x41800000, which is the float 16 + q,
// exactly. A byte permute builds that float from a pre-shifted copy of the word, so each weight
// costs 1.5 integer instructions and half a packed FMA and never touches the conversion unit.
// The dot product accumulates sum((16 + q) * x); callers remove the offset with the chunk's
// sum of x:  sum(q * x) = acc - 16 * sum(x), folded into the group's min term.
//
// xp[0..3] hold (x0,x1), (x2,x3), (x4,x5), (x6,x7) for the word's nibbles in k order.
DRB_DEV unsigned long long dot8_q4(uint32_t w, const unsigned long long* xp, unsigned long long acc) {
  const uint32_t ev = lop3_and_or(w << 3, 0x78787878u, 0x80808080u);  // nibbles 0,2,4,6 as 0x80|q<<3
  const uint32_t od = lop3_and_or(w >> 1, 0x78787878u, 0x80808080u);  // nibbles 1,3,5,7
  const uint32_t hi = 0x00000041u;                                    // byte 4 = 0x41, byte 5 = 0x00
  acc = fma2(pack2(__uint_as_float(prmt(ev, hi, 0x4055u)), __uint_as_float(prmt(od, hi, 0x4055u))), xp[0], acc);
  acc = fma2(pack2(__uint_as_float(prmt(ev, hi, 0x4155u)), __uint_as_float(prmt(od, hi, 0x4155u))), xp[1], acc);
  acc = fma2(pack2(__uint_as_float(prmt(ev, hi, 0x4255u)), __uint_as_float(prmt(od, hi, 0x4255u))), xp[2], acc);
  acc = fma2(pack2(__uint_as_float(prmt(ev, hi, 0x4355u)), __uint_as_float(prmt(od, hi, 0x4355u))), xp[3], acc);
  return acc;
}

// One 16-byte chunk (32 nibbles, k ascending) against xp[0..15]; returns sum((16 + q) * x).
DRB_DEV float dot32_q4(const uint4& v, const unsigned long long* xp) {
  unsigned long long a = 0ull, b = 0ull;
  a = dot8_q4(v.x, xp + 0, a);
  b = dot8_q4(v.y, xp + 4, b);
  a = dot8_q4(v.z, xp + 8, a);
  b = dot8_q4(v.w, xp + 12, b);
  float a0, a1, b0, b1;
  unpack2(a, a0, a1);
  unpack2(b, b0, b1);
  return (a0 + a1) + (b0 + b1);
}

// ------------------------------------------------------------------------------------------
// int8: four signed bytes of one word against four activations.
//
// Flipping the sign bit gives u = b + 128 in 0..255; a byte permute builds 0x4B0000uu, the float
// 2^23 + u; one packed add removes 2^23 + 128 exactly. 2.25 instructions per weight.
DRB_DEV unsigned long long dot4_q8(uint32_t w, const unsigned long long* xp, unsigned long long acc) {
  const uint32_t u = w ^ 0x80808080u;
  const uint32_t hi = 0x0000004Bu;
  const unsigned long long off = pack2(-8388736.f, -8388736.f);  // -(2^23 + 128)
  const unsigned long long p0 = add2(pack2(__uint_as_float(prmt(u, hi, 0x4550u)), __uint_as_float(prmt(u, hi, 0x4551u))), off);
  const unsigned long long p1 = add2(pack2(__uint_as_float(prmt(u, hi, 0x4552u)), __uint_as_float(prmt(u, hi, 0x4553u))), off);
  acc = fma2(p0, xp[0], acc);
  acc = fma2(p1, xp[1], acc);
  return acc;
}

// One 16-byte chunk (16 int8, k ascending) against xp[0..7]; returns sum(w * x).
DRB_DEV float dot16_q8(const uint4& v, const unsigned long long* xp) {
  unsigned long long a = 0ull, b = 0ull;
  a = dot4_q8(v.x, xp + 0, a);
  b = dot4_q8(v.y, xp + 2, b);
  a = dot4_q8(v.z, xp + 4, a);
  b = dot4_q8(v.w, xp + 6, b);
  float a0, a1, b0, b1;
  unpack2(a, a0, a1);
  unpack2(b, b0, b1);
  return (a0 + a1) + (b0 + b1);
}

// One 16-byte chunk of bf16 (8 weights) against xp[0..3].
DRB_DEV unsigned long long dot8_bf16(const uint4& v, const unsigned long long* xp, unsigned long long acc) {
  acc = fma2(pack2(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u)), xp[0], acc);
  acc = fma2(pack2(__uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u)), xp[1], acc);
  acc = fma2(pack2(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u)), xp[2], acc);
  acc = fma2(pack2(__uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u)), xp[3], acc);
  return acc;
}

// ------------------------------------------------------------------------------------------
// Integer dot products (dp4a). A lane's slice of the activation vector is re-expressed once per
// kernel as block fixed point: x_k = delta * n_k with |n_k| <= 2^20 and delta = max|x| * 2^-20 over
// the slice, n_k split into three signed limbs n = l0 + 128 l1 + 16384 l2 (l0, l1 in [-64, 63]).
// A weight word then costs one dp4a per limb, four multiply-adds each, accumulated exactly in
// int32; the three sums are recombined and converted to fp32 once per 16-byte chunk.
// Quantisation error of an activation is at most delta / 2 = 2^-21 of the slice's largest value
// (fp32 itself carries 2^-24 of each value), and nothing is rounded during accumulation.

DRB_DEV int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
}
DRB_DEV int dp4a_ss(uint32_t a_s8x4, uint32_t b_s8x4, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8x4), "r"(b_s8x4), "r"(c));
  return d;
}

// Splits n (|n| <= 2^20 + a little) into its three limbs.
DRB_DEV void limbs3(int n, int& l0, int& l1, int& l2) {
  l0 = ((n + 64) & 127) - 64;
  const int n1 = (n - l0) >> 7;
  l1 = ((n1 + 64) & 127) - 64;
  l2 = (n1 - l1) >> 7;
}

// N consecutive activations held by one lane, as limbs packed four to a word.
//   NATURAL order: word i of limb j holds k = 4i .. 4i+3                     (int8 weight words)
//   EVEN/ODD order (EO): word i holds k = 8(i/2) + {0,2,4,6} for even i and {1,3,5,7} for odd i,
//   which is how the low and the high nibbles of an int4 weight word line up.
template <int N, bool EO>
struct QAct {
  uint32_t l[3][N / 4];
  float delta;
  DRB_DEV void quantize(const float* x) {
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < N; ++k) m = fmaxf(m, fabsf(x[k]));
    delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
    const float inv = 1.f / delta;
#pragma unroll
    for (int j = 0; j < 3; ++j)
#pragma unroll
      for (int i = 0; i < N / 4; ++i) l[j][i] = 0u;
#pragma unroll
    for (int k = 0; k < N; ++k) {
      int l0, l1, l2;
      limbs3(__float2int_rn(x[k] * inv), l0, l1, l2);
      const int word = EO ? 2 * (k / 8) + (k & 1) : k / 4;
      const int byte = EO ? (k & 7) >> 1 : k & 3;
      l[0][word] |= (uint32_t)(l0 & 0xff) << (8 * byte);
      l[1][word] |= (uint32_t)(l1 & 0xff) << (8 * byte);
      l[2][word] |= (uint32_t)(l2 & 0xff) << (8 * byte);
    }
  }
};

// Cooperative quantisation: instead of every lane converting its own slice (hundreds of
// instructions, repeated by every warp that owns the same slice), each thread converts the float4
// it loaded, the threads of one block of 16 or 32 values agree on max|x| with shuffles, and the
// packed limb words go to shared memory, from where the owning lanes pick them up with a few
// 128-bit loads. Must be called by whole warps (it shuffles); threads with nothing to convert pass
// valid = false. g4 is the float4's index in the vector: consecutive lanes hold consecutive g4.
//
// Even/odd packing, 32 values per block, 112 bytes per block: 3 limbs x 8 words, delta, sum(x), pad
// (the 112-byte stride keeps the lanes' 128-bit reads on distinct banks).
constexpr int QB32_BYTES = 112;
DRB_DEV void quant_store_eo(unsigned char* blocks, int g4, float4 v, bool valid) {
  float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
  }
  if (!valid) return;
  const float delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
  const float inv = 1.f / delta;
  int l[4][3];
  limbs3(__float2int_rn(v.x * inv), l[0][0], l[0][1], l[0][2]);
  limbs3(__float2int_rn(v.y * inv), l[1][0], l[1][1], l[1][2]);
  limbs3(__float2int_rn(v.z * inv), l[2][0], l[2][1], l[2][2]);
  limbs3(__float2int_rn(v.w * inv), l[3][0], l[3][1], l[3][2]);
  unsigned char* blk = blocks + (size_t)(g4 >> 3) * QB32_BYTES;
  const int sub = g4 & 1, w = 2 * ((g4 & 7) >> 1);
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    *reinterpret_cast<uint16_t*>(blk + (j * 8 + w) * 4 + 2 * sub) = (uint16_t)((l[0][j] & 0xff) | ((l[2][j] & 0xff) << 8));
    *reinterpret_cast<uint16_t*>(blk + (j * 8 + w + 1) * 4 + 2 * sub) = (uint16_t)((l[1][j] & 0xff) | ((l[3][j] & 0xff) << 8));
  }
  if ((g4 & 7) == 0) {
    *reinterpret_cast<float*>(blk + 96) = delta;
    *reinterpret_cast<float*>(blk + 100) = sum;
  }
}

// Natural packing, 16 values per block, 64 bytes per block: 3 limbs x 4 words, delta, pad.
constexpr int QB16_BYTES = 64;
DRB_DEV void quant_store_nat(unsigned char* blocks, int g4, float4 v, bool valid) {
  float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  if (!valid) return;
  const float delta = m > 0.f ? m * (1.f / 1048576.f) : 1.f;
  const float inv = 1.f / delta;
  int l[4][3];
  limbs3(__float2int_rn(v.x * inv), l[0][0], l[0][1], l[0][2]);
  limbs3(__float2int_rn(v.y * inv), l[1][0], l[1][1], l[1][2]);
  limbs3(__float2int_rn(v.z * inv), l[2][0], l[2][1], l[2][2]);
  limbs3(__float2int_rn(v.w * inv), l[3][0], l[3][1], l[3][2]);
  unsigned char* blk = blocks + (size_t)(g4 >> 2) * QB16_BYTES;
#pragma unroll
  for (int j = 0; j < 3; ++j)
    *reinterpret_cast<uint32_t*>(blk + (j * 4 + (g4 & 3)) * 4) =
        (uint32_t)(l[0][j] & 0xff) | ((uint32_t)(l[1][j] & 0xff) << 8) | ((uint32_t)(l[2][j] & 0xff) << 16) | ((uint32_t)(l[3][j] & 0xff) << 24);
  if ((g4 & 3) == 0) *reinterpret_cast<float*>(blk + 48) = delta;
}

DRB_DEV void qact_load(QAct<32, true>& a, float& sum, const unsigned char* blk) {
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    const uint4 v = reinterpret_cast<const uint4*>(blk)[i];
    a.l[i / 2][(i & 1) * 4 + 0] = v.x, a.l[i / 2][(i & 1) * 4 + 1] = v.y, a.l[i / 2][(i & 1) * 4 + 2] = v.z, a.l[i / 2][(i & 1) * 4 + 3] = v.w;
  }
  a.delta = *reinterpret_cast<const float*>(blk + 96);
  sum = *reinterpret_cast<const float*>(blk + 100);
}

DRB_DEV void qact_load(QAct<16, false>& a, const unsigned char* blk) {
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const uint4 v = reinterpret_cast<const uint4*>(blk)[j];
    a.l[j][0] = v.x, a.l[j][1] = v.y, a.l[j][2] = v.z, a.l[j][3] = v.w;
  }
  a.delta = *reinterpret_cast<const float*>(blk + 48);
}

// 32 int4 products: |sum| <= 32 * 15 * 2^20 < 2^29, the integer recombination cannot overflow.
DRB_DEV float recombine(int a0, int a1, int a2) { return (float)(a0 + (a1 << 7) + (a2 << 14)); }
// int8 weights: 32 products of magnitude up to 128 * 2^20 reach 2^32 (a constant slice against weights of one
// sign does it), so the top limb's sum joins in fp32. |a0| + |a1 << 7| < 2^26 stays an integer sum; a2 is below
// 2^19 and exact as a float; the one rounding is 2^-24 of the result, as every fp32 sum has.
DRB_DEV float recombine_wide(int a0, int a1, int a2) { return fmaf((float)a2, 16384.f, (float)(a0 + (a1 << 7))); }

// sum_k q_k n_k over one 16-byte chunk of int4 weights (32 nibbles, k ascending) against words
// [w0, w0 + 8) of an even/odd-ordered slice. Multiply by delta (and the group scale) afterwards.
template <int N>
DRB_DEV float dot32_q4_i(const uint4& v, const QAct<N, true>& a, int w0) {
  int a0 = 0, a1 = 0, a2 = 0;
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
    a0 = dp4a_us(lo, a.l[0][w0 + 2 * i], a0), a0 = dp4a_us(hi, a.l[0][w0 + 2 * i + 1], a0);
    a1 = dp4a_us(lo, a.l[1][w0 + 2 * i], a1), a1 = dp4a_us(hi, a.l[1][w0 + 2 * i + 1], a1);
    a2 = dp4a_us(lo, a.l[2][w0 + 2 * i], a2), a2 = dp4a_us(hi, a.l[2][w0 + 2 * i + 1], a2);
  }
  return recombine(a0, a1, a2);
}

// sum_k w_k n_k over one 16-byte chunk of int8 weights against words [w0, w0 + 4) of a natural-ordered slice.
template <int N>
DRB_DEV float dot16_q8_i(const uint4& v, const QAct<N, false>& a, int w0) {
  int a0 = 0, a1 = 0, a2 = 0;
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a0 = dp4a_ss(w[i], a.l[0][w0 + i], a0);
    a1 = dp4a_ss(w[i], a.l[1][w0 + i], a1);
    a2 = dp4a_ss(w[i], a.l[2][w0 + i], a2);
  }
  return recombine_wide(a0, a1, a2);
}

// The same for an even/odd-ordered slice: two weight words are first regrouped into their even and odd bytes.
// Covers two 16-byte chunks (32 int8, k ascending) against words [w0, w0 + 8).
template <int N>
DRB_DEV float dot32_q8_eo(const uint4& v0, const uint4& v1, const QAct<N, true>& a, int w0) {
  int a0 = 0, a1 = 0, a2 = 0;
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t ev = prmt(w[2 * i], w[2 * i + 1], 0x6420u), od = prmt(w[2 * i], w[2 * i + 1], 0x7531u);
    a0 = dp4a_ss(ev, a.l[0][w0 + 2 * i], a0), a0 = dp4a_ss(od, a.l[0][w0 + 2 * i + 1], a0);
    a1 = dp4a_ss(ev, a.l[1][w0 + 2 * i], a1), a1 = dp4a_ss(od, a.l[1][w0 + 2 * i + 1], a1);
    a2 = dp4a_ss(ev, a.l[2][w0 + 2 * i], a2), a2 = dp4a_ss(od, a.l[2][w0 + 2 * i + 1], a2);
  }
  return recombine_wide(a0, a1, a2);
}

// ------------------------------------------------------------------------------------------
// host-side launch helper

// Launches with the programmatic-stream-serialization attribute when `pdl` is set, so the kernel
// may start while its predecessor drains; the kernel itself calls pdl_wait() before it touches
// anything the predecessor wrote.
template <typename... KArgs, typename... Args>
static inline cudaError_t drb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Per-device setup (see runtime.cuh): attributes that must be set before a kernel's first launch and
// the scratch words of the grid-wide barriers. Set up by the pre-capture hooks (dr_stream_create,
// dr_malloc, dr_cublas_create, dr_sample_init) or lazily by the first launcher call on a stream that
// is not capturing; a first call inside a capture finds ready == false and the launcher returns -2.
struct DrbDevice {
  int sms;              // blocks of a persistent grid: the multiprocessor count
  bool pdl;             // programmatic dependent launch enabled (DRB_PDL=0 turns it off)
  bool ready;           // attributes set
};
const DrbDevice& drb_device(cudaStream_t st);
