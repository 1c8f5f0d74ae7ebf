// Checkpoint quantisers on the GPU: the reference's converter (tools/convert.py) turns bf16/fp8 expert weights
// into the int4 / int8 layouts the kernels stream. These two kernels restate its per-group procedures operation by
// operation in IEEE fp32 (no fused multiply-add, round-to-nearest division, fp16 rounding of scale and min), so that
// codes and scales come out as the reference writes them. That includes the ORDER of the 64-term sums that decide
// between two clipping candidates: eight running sums over the inputs 8 i + j (i ascending), then
// ((r0 + r1) + (r2 + r3)) + ((r4 + r5) + (r6 + r7)): the order of the CPU restatement of the converter, which
// reproduces the converter's own output on the committed fixture bit for bit. (The converter's sums are a library's
// vectorised reduction whose exact order depends on the host's vector width; where two candidates' errors agree to
// the last bit, its pick is not defined by its source.)
//
//   drb_quant_q4: tools/convert.py:44-89 (`quant_q4_groups`: 24-step clipping search, least-squares refit) and
//                 92-101 (`quant_q4`: packing, low nibble = even k). One warp per group of 64 inputs.
//   drb_quant_q8: tools/convert.py:33-41 (`quant_q8`). One warp per group of 128 inputs.
#pragma once

#include "common.cuh"

namespace quant {

constexpr int STEPS = 24;
// float32(1.0 - 0.5 * i / 24), the reference's shrink factors
__constant__ float c_shrink[STEPS] = {1.0f,        0.97916669f, 0.95833331f, 0.9375f,     0.91666669f, 0.89583331f, 0.875f,      0.85416669f,
                                      0.83333331f, 0.8125f,     0.79166669f, 0.77083331f, 0.75f,       0.72916669f, 0.70833331f, 0.6875f,
                                      0.66666669f, 0.64583331f, 0.625f,      0.60416669f, 0.58333331f, 0.5625f,     0.54166669f, 0.52083331f};

DRB_DEV float half_round(float v) { return __half2float(__float2half_rn(v)); }

// Sum of the group's 64 values in the converter's order; lane l passes inputs 2l (a) and 2l + 1 (b), every lane
// gets the total. Running sum j collects inputs j, 8 + j, 16 + j, ...: those of lanes j / 2, j / 2 + 4, ...
DRB_DEV float sum64(float a, float b) {
  const int p = threadIdx.x & 3;
  float r0 = __shfl_sync(0xffffffffu, a, p), r1 = __shfl_sync(0xffffffffu, b, p);  // running sums 2p and 2p + 1
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    r0 = __fadd_rn(r0, __shfl_sync(0xffffffffu, a, p + 4 * i));
    r1 = __fadd_rn(r1, __shfl_sync(0xffffffffu, b, p + 4 * i));
  }
  const float pr = __fadd_rn(r0, r1);                                       // r[2p] + r[2p + 1]
  const float q = __fadd_rn(__shfl_sync(0xffffffffu, pr, 0), __shfl_sync(0xffffffffu, pr, 1));  // (r0 + r1) + (r2 + r3)
  const float h = __fadd_rn(__shfl_sync(0xffffffffu, pr, 2), __shfl_sync(0xffffffffu, pr, 3));  // (r4 + r5) + (r6 + r7)
  return __fadd_rn(q, h);
}

// Lane l holds inputs 2l and 2l + 1 of the group.
__global__ void __launch_bounds__(256) k_quant_q4(const float* __restrict__ w, size_t groups, uint8_t* __restrict__ q,
                                                  __half2* __restrict__ sm) {
  const size_t g = (size_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (g >= groups) return;
  const float2 v = reinterpret_cast<const float2*>(w + g * 64)[lane];
  float gmin = fminf(v.x, v.y), gmax = fmaxf(v.x, v.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    gmin = fminf(gmin, __shfl_xor_sync(0xffffffffu, gmin, o));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
  }
  const float center = __fmul_rn(__fadd_rn(gmin, gmax), 0.5f);
  float best_err = 0.f, best_scale = 0.f, best_lo = 0.f, bq0 = 0.f, bq1 = 0.f;
  for (int i = 0; i < STEPS; ++i) {
    const float shrink = c_shrink[i];
    const float lo_c = __fadd_rn(center, __fmul_rn(__fsub_rn(gmin, center), shrink));
    const float hi_c = __fadd_rn(center, __fmul_rn(__fsub_rn(gmax, center), shrink));
    const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi_c, lo_c), 15.0f), 1e-10f);
    const float scale_h = fmaxf(half_round(scale), 1e-10f);
    const float lo_h = half_round(lo_c);
    const float q0 = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v.x, lo_h), scale_h)), 0.f), 15.f);
    const float q1 = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v.y, lo_h), scale_h)), 0.f), 15.f);
    const float d0 = __fsub_rn(__fadd_rn(__fmul_rn(q0, scale_h), lo_h), v.x);
    const float d1 = __fsub_rn(__fadd_rn(__fmul_rn(q1, scale_h), lo_h), v.y);
    const float err = sum64(__fmul_rn(d0, d0), __fmul_rn(d1, d1));
    if (i == 0 || err < best_err) best_err = err, best_scale = scale_h, best_lo = lo_h, bq0 = q0, bq1 = q1;
  }
  // One least-squares refinement of (scale, min) given the codes.
  const float n = 64.f;
  const float sq = sum64(bq0, bq1);
  const float sqq = sum64(__fmul_rn(bq0, bq0), __fmul_rn(bq1, bq1));
  const float sw = sum64(v.x, v.y);
  const float sqw = sum64(__fmul_rn(bq0, v.x), __fmul_rn(bq1, v.y));
  const float det = __fsub_rn(__fmul_rn(n, sqq), __fmul_rn(sq, sq));
  const bool ok = fabsf(det) > 1e-6f;
  const float ls_scale = ok ? __fdiv_rn(__fsub_rn(__fmul_rn(n, sqw), __fmul_rn(sq, sw)), det) : best_scale;
  const float ls_min = ok ? __fdiv_rn(__fsub_rn(sw, __fmul_rn(ls_scale, sq)), n) : best_lo;
  const float ls_scale_h = half_round(ls_scale), ls_min_h = half_round(ls_min);
  const float e0 = __fsub_rn(__fadd_rn(__fmul_rn(bq0, ls_scale_h), ls_min_h), v.x);
  const float e1 = __fsub_rn(__fadd_rn(__fmul_rn(bq1, ls_scale_h), ls_min_h), v.y);
  const float ls_err = sum64(__fmul_rn(e0, e0), __fmul_rn(e1, e1));
  if (ls_err < best_err && ok && ls_scale_h > 0.f) best_scale = ls_scale_h, best_lo = ls_min_h;
  q[g * 32 + lane] = (uint8_t)((unsigned)bq0 | ((unsigned)bq1 << 4));
  if (lane == 0) sm[g] = __halves2half2(__float2half_rn(best_scale), __float2half_rn(best_lo));
}

// Lane l holds inputs 4l .. 4l + 3 of the group of 128.
__global__ void __launch_bounds__(256) k_quant_q8(const float* __restrict__ w, size_t groups, int8_t* __restrict__ q,
                                                  __half* __restrict__ s) {
  const size_t g = (size_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (g >= groups) return;
  const float4 v = reinterpret_cast<const float4*>(w + g * 128)[lane];
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-12f);
  const float scale = fmaxf(half_round(__fdiv_rn(amax, 127.0f)), 1e-12f);
  auto code = [&](float x) { return (int)fminf(fmaxf(rintf(__fdiv_rn(x, scale)), -127.f), 127.f); };
  const char4 o = make_char4((signed char)code(v.x), (signed char)code(v.y), (signed char)code(v.z), (signed char)code(v.w));
  reinterpret_cast<char4*>(q + g * 128)[lane] = o;
  if (lane == 0) s[g] = __float2half_rn(scale);
}

}  // namespace quant

// w: groups x 64 consecutive floats (a [E, N, K] tensor with K a multiple of 64, row-major). q: groups x 32 bytes,
// sm: groups x (scale, min) f16: the layouts of `moe.*.q4` / `moe.*.sm`. No counterpart in the reference's C ABI
// (its quantiser is the Python converter).
extern "C" int drb_quant_q4(const float* w, size_t groups, uint8_t* q, __half2* sm, cudaStream_t st) {
  if (groups == 0) return 0;
  quant::k_quant_q4<<<(unsigned)((groups + 7) / 8), 256, 0, st>>>(w, groups, q, sm);
  return 0;
}

// w: groups x 128 consecutive floats; q: the int8 codes; s: one f16 scale per group (`*.q8` / `*.s`).
extern "C" int drb_quant_q8(const float* w, size_t groups, int8_t* q, __half* s, cudaStream_t st) {
  if (groups == 0) return 0;
  quant::k_quant_q8<<<(unsigned)((groups + 7) / 8), 256, 0, st>>>(w, groups, q, s);
  return 0;
}
