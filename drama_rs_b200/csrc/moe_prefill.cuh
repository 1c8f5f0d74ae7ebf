// Prefill-side kernels of the MoE path: per-row routing bookkeeping (count / permute / combine),
// the expert-grouped int4 "GEMM" (dr_moe_prefill), and the elementwise helpers the reference's
// prefill calls around cuBLAS (dequant_q8, f32_to_bf16, swiglu_rows, rmsnorm).
//
// Replaces kernels/drama.cu:744-968 and 1114-1202 of the reference, same C signatures
// (src/ffi.rs:61-77).
#pragma once

#include "common.cuh"

namespace pf {

constexpr int H = 2048, I = 512;

// ------------------------------------------------------------------------------------------
// bookkeeping

__global__ void k_count(const int* __restrict__ idx, int n, int* __restrict__ counts) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) atomicAdd(counts + idx[i], 1);
}

// One block per (row, k) pair: claim the next slot of the pair's expert, remember it, copy the row.
__global__ void __launch_bounds__(128)
    k_permute(const int* __restrict__ idx, int topk, const int* __restrict__ offsets, int* __restrict__ fill,
              int* __restrict__ slot_of, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xp, int Hd) {
  pdl_wait();
  const int i = blockIdx.x;
  __shared__ int slot;
  if (threadIdx.x == 0) {
    const int e = idx[i];
    slot = offsets[e] + atomicAdd(fill + e, 1);
    slot_of[i] = slot;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / topk) * Hd);
  uint4* dst = reinterpret_cast<uint4*>(xp + (size_t)slot * Hd);
  for (int c = threadIdx.x; c < Hd / 8; c += blockDim.x) dst[c] = src[c];
}

// x[r] += sigmoid(sgate[r]) * shared[r] + sum_k w[r,k] * Y[slot_of[r,k]], k ascending (fixed order, so
// the result does not depend on how slots were handed out).
__global__ void __launch_bounds__(256)
    k_combine(float* __restrict__ x, const float* __restrict__ Y, const int* __restrict__ slot_of,
              const float* __restrict__ wts, const float* __restrict__ sgate, const float* __restrict__ shared, int topk,
              int Hd) {
  pdl_wait();
  const int r = blockIdx.x;
  const float sg = sigmoid_f(sgate[r]);
  for (int c = threadIdx.x * 4; c < Hd; c += blockDim.x * 4) {
    const float4 sh = *reinterpret_cast<const float4*>(shared + (size_t)r * Hd + c);
    float4 acc = make_float4(sg * sh.x, sg * sh.y, sg * sh.z, sg * sh.w);
    for (int k = 0; k < topk; ++k) {
      const float w = wts[r * topk + k];
      const float4 v = *reinterpret_cast<const float4*>(Y + (size_t)slot_of[r * topk + k] * Hd + c);
      acc.x += w * v.x, acc.y += w * v.y, acc.z += w * v.z, acc.w += w * v.w;
    }
    float4* xo = reinterpret_cast<float4*>(x + (size_t)r * Hd + c);
    float4 o = *xo;
    o.x += acc.x, o.y += acc.y, o.z += acc.z, o.w += acc.w;
    *xo = o;
  }
}

// ------------------------------------------------------------------------------------------
// expert-grouped int4 contraction on CUDA cores.
//
// Rows of xp are sorted by expert. A block owns 16 (gate, up) row pairs (gate/up kernel) or 32 output
// rows (down kernel) of one expert, keeps those weight rows packed in registers for its whole
// life, and walks the expert's tokens; the weights are read from memory once per block.
// The intermediate is kept in fp16 (the buffer is 16 bits per element by the ABI; fp16 carries three
// more mantissa bits than bf16 at these magnitudes, which the 1e-3 output tolerance needs).

__global__ void __launch_bounds__(256)
    k_pf_gate_up(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const __nv_bfloat16* __restrict__ xp,
                 const int* __restrict__ offsets, const int* __restrict__ counts, __half* __restrict__ act) {
  pdl_wait();
  const int e = blockIdx.x;
  const int cnt = counts[e];
  if (cnt == 0) return;
  const int off = offsets[e];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j0 = (blockIdx.y * 8 + warp) * 2;
  const uint8_t* q = Q + (size_t)e * (2 * I) * (H / 2);
  const __half2* sm = SM + (size_t)e * (2 * I) * (H / 64);
  // rows: r = 0,1 -> gate j0, j0+1 ; r = 2,3 -> up j0, j0+1. Chunks lane and lane+32 of each.
  uint4 w[4][2];
  float2 s[4][2];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const size_t row = (size_t)(r >> 1) * I + j0 + (r & 1);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      w[r][h] = __ldg(reinterpret_cast<const uint4*>(q + row * (H / 2)) + lane + 32 * h);
      s[r][h] = __half22float2(sm[row * (H / 64) + 16 * h + (lane >> 1)]);
    }
  }
  for (int t = 0; t < cnt; ++t) {
    const __nv_bfloat16* xr = xp + (size_t)(off + t) * H;
    unsigned long long xv[32];
    float X[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr + h * 1024 + 32 * lane) + c);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = __uint_as_float(u[i] << 16), b = __uint_as_float(u[i] & 0xffff0000u);
          xv[h * 16 + c * 4 + i] = pack2(a, b);
          sum += a + b;
        }
      }
      X[h] = sum;
    }
    float d[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      d[r] = s[r][0].x * dot32_q4(w[r][0], xv) + (s[r][0].y - 16.f * s[r][0].x) * X[0] +
             s[r][1].x * dot32_q4(w[r][1], xv + 16) + (s[r][1].y - 16.f * s[r][1].x) * X[1];
      d[r] = warp_sum(d[r]);
    }
    if (lane < 2) act[(size_t)(off + t) * I + j0 + lane] = __float2half_rn(silu_f(lane ? d[1] : d[0]) * (lane ? d[3] : d[2]));
  }
}

__global__ void __launch_bounds__(256)
    k_pf_down(const uint8_t* __restrict__ Q, const __half2* __restrict__ SM, const __half* __restrict__ act,
              const int* __restrict__ offsets, const int* __restrict__ counts, float* __restrict__ y) {
  pdl_wait();
  const int e = blockIdx.x;
  const int cnt = counts[e];
  if (cnt == 0) return;
  const int off = offsets[e];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cc = lane & 15, half = lane >> 4;
  const int n0 = (blockIdx.y * 8 + warp) * 4;
  const uint8_t* q = Q + (size_t)e * H * (I / 2);
  const __half2* sm = SM + (size_t)e * H * (I / 64);
  uint4 w[2];
  float2 s[2];
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const size_t row = n0 + 2 * p + half;
    w[p] = __ldg(reinterpret_cast<const uint4*>(q + row * (I / 2)) + cc);
    s[p] = __half22float2(sm[row * (I / 64) + (cc >> 1)]);
  }
  for (int t = 0; t < cnt; ++t) {
    const __half* ar = act + (size_t)(off + t) * I + 32 * cc;
    unsigned long long av[16];
    float A = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(ar) + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
        av[c * 4 + i] = pack2(f.x, f.y);
        A += f.x + f.y;
      }
    }
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float v = s[p].x * dot32_q4(w[p], av) + (s[p].y - 16.f * s[p].x) * A;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (cc == 0) y[(size_t)(off + t) * H + n0 + 2 * p + half] = v;
    }
  }
}

// ------------------------------------------------------------------------------------------
// elementwise

__global__ void k_dequant_q8(const int8_t* __restrict__ W, const __half* __restrict__ S, __nv_bfloat16* __restrict__ out,
                             size_t n_elems, int K) {
  pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
  if (i >= n_elems) return;
  const size_t row = i / K, col = i % K;
  const float s = __half2float(S[row * (K / 128) + col / 128]);
  const uint4 v = *reinterpret_cast<const uint4*>(W + i);
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
  __align__(16) __nv_bfloat16 o[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j] = __float2bfloat16((float)(int8_t)(u[j >> 2] >> (8 * (j & 3))) * s);
  reinterpret_cast<uint4*>(out + i)[0] = reinterpret_cast<uint4*>(o)[0];
  reinterpret_cast<uint4*>(out + i)[1] = reinterpret_cast<uint4*>(o)[1];
}

__global__ void k_f32_to_bf16(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16(x[i]);
}

// y[r, j] = silu(h[r, j]) * h[r, I + j] in bf16; h has row stride 2I.
__global__ void k_swiglu_rows(const float* __restrict__ h, __nv_bfloat16* __restrict__ y, int rows, int Id) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * Id) return;
  const size_t r = i / Id, j = i % Id;
  y[i] = __float2bfloat16(silu_f(h[r * 2 * Id + j]) * h[r * 2 * Id + Id + j]);
}

// Row-wise RMSNorm ("+1" already folded into w). Writes f32 and/or bf16.
__global__ void __launch_bounds__(256)
    k_rmsnorm(const float* __restrict__ x, const float* __restrict__ w, float* y, __nv_bfloat16* yb, int D, float eps) {
  pdl_wait();
  __shared__ float red[9];
  const float* xr = x + (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) ss += xr[i] * xr[i];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    red[8] = rsqrtf(t / D + eps);
  }
  __syncthreads();
  const float inv = red[8];
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = xr[i] * inv * w[i];
    if (y) y[(size_t)blockIdx.x * D + i] = v;
    if (yb) yb[(size_t)blockIdx.x * D + i] = __float2bfloat16(v);
  }
}

// Router logits whose value for a row does not depend on how many rows are computed together: every (row, output)
// pair is one warp's dot product in a fixed order (lane l takes the 16-byte chunks l, l + 32, ... of the K = 2048
// inputs, products exact in fp32, one fixed butterfly). A library GEMM picks its kernel by the batch size (measured:
// logits of the same row differ by 1.2e-6 between a batch of 300 and a batch of 38), which would let the routing of
// a row depend on how the rows are spread over the GPUs. Block (x, y) = RB rows x the outputs y, y + gridDim.y, ...;
// its warp w takes every 8th of those. The split over y only adds parallelism: it does not change any sum.
constexpr int RL_RB = 4, RL_K = 2048, RL_SPLIT = 9;
__global__ void __launch_bounds__(256)
    k_router_logits(const __nv_bfloat16* __restrict__ xb, const __nv_bfloat16* __restrict__ w, float* __restrict__ logits,
                    int rows, int e1, float beta) {
  pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 xs[RL_RB][RL_K];
  const int r0 = blockIdx.x * RL_RB;
  const int nr = min(RL_RB, rows - r0);
  for (int i = threadIdx.x; i < RL_RB * RL_K / 8; i += blockDim.x) {
    const int r = i / (RL_K / 8), c = i % (RL_K / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < nr) v = __ldcg(reinterpret_cast<const uint4*>(xb + (size_t)(r0 + r) * RL_K) + c);
    reinterpret_cast<uint4*>(&xs[r][0])[c] = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = blockIdx.y + gridDim.y * warp; o < e1; o += gridDim.y * 8) {
    const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)o * RL_K);
    uint4 wv8[RL_K / 8 / 32];
#pragma unroll
    for (int j = 0; j < RL_K / 8 / 32; ++j) wv8[j] = __ldg(wr + lane + 32 * j);  // all eight in flight at once
    float acc[RL_RB];
#pragma unroll
    for (int r = 0; r < RL_RB; ++r) acc[r] = 0.f;
#pragma unroll
    for (int j = 0; j < RL_K / 8 / 32; ++j) {
      const uint4 wv = wv8[j];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int r = 0; r < RL_RB; ++r) {
        const uint4 xv = reinterpret_cast<const uint4*>(&xs[r][0])[lane + 32 * j];
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          acc[r] = fmaf(__uint_as_float(ww[t] << 16), __uint_as_float(xw[t] << 16), acc[r]);
          acc[r] = fmaf(__uint_as_float(ww[t] & 0xffff0000u), __uint_as_float(xw[t] & 0xffff0000u), acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RL_RB; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && r < nr) {
        float* out = logits + (size_t)(r0 + r) * e1 + o;
        *out = beta != 0.f ? fmaf(beta, *out, v) : v;
      }
    }
  }
}

// offsets[e] = sum of counts[0..e): the exclusive scan the reference does on the host between two launches
// (src/engine.rs:567-574). One block, any number of experts.
__global__ void __launch_bounds__(256) k_offsets(const int* __restrict__ counts, int E, int* __restrict__ offsets) {
  pdl_wait();
  __shared__ int warp_tot[8];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < E; base += 256) {
    const int i = base + threadIdx.x;
    const int c = i < E ? counts[i] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (i < E) offsets[i] = before + incl - c;
    __syncthreads();
    if (threadIdx.x == 255) carry = before + incl;
    __syncthreads();
  }
}

static cudaError_t configure_all() {
  cudaError_t e;
  if ((e = drb_carveout(k_offsets)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_router_logits)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_count)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_permute)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_combine)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_pf_gate_up)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_pf_down)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_dequant_q8)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_f32_to_bf16)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_swiglu_rows)) != cudaSuccess) return e;
  return drb_carveout(k_rmsnorm);
}

}  // namespace pf

// Reference: kernels/drama.cu:750-753; src/ffi.rs:65. counts must be zeroed by the caller.
extern "C" int dr_moe_count(const int* idx, int n, int* counts, cudaStream_t st) {
  if (n <= 0) return 0;
  pf::k_count<<<(n + 255) / 256, 256, 0, st>>>(idx, n, counts);
  return 0;
}

// No counterpart in the reference, which downloads the counts and scans them on the host (src/engine.rs:567-574):
// with this call the prefill sequence needs no host round trip and can be captured in a graph.
extern "C" int drb_moe_offsets(const int* counts, int e, int* offsets, cudaStream_t st) {
  if (e <= 0) return 0;
  pf::k_offsets<<<1, 256, 0, st>>>(counts, e, offsets);
  return 0;
}

// logits [rows, e1] = xb [rows, h] . w [e1, h]^T + beta * logits, with per-row results that do not depend on `rows`
// (see k_router_logits). The reference computes these logits with cublasGemmEx (src/engine.rs:554); this call is for
// hosts that spread rows over several GPUs and need the same routing at every split. h == 2048, else -1.
extern "C" int drb_router_logits(const __nv_bfloat16* xb, const __nv_bfloat16* w, float* logits, int rows, int e1, int h,
                                 float beta, cudaStream_t st) {
  if (h != pf::RL_K) return -1;
  if (rows <= 0 || e1 <= 0) return 0;
  pf::k_router_logits<<<dim3((rows + pf::RL_RB - 1) / pf::RL_RB, pf::RL_SPLIT), 256, 0, st>>>(xb, w, logits, rows, e1, beta);
  return 0;
}

// Reference: kernels/drama.cu:774-778; src/ffi.rs:66-69. fill must be zeroed by the caller.
extern "C" int dr_moe_permute(const int* idx, int rows, int topk, const int* offsets, int* fill, int* slot_of,
                              const __nv_bfloat16* x, __nv_bfloat16* xp, int H, cudaStream_t st) {
  if (H % 8 != 0) return -1;
  if (rows * topk <= 0) return 0;
  pf::k_permute<<<rows * topk, 128, 0, st>>>(idx, topk, offsets, fill, slot_of, x, xp, H);
  return 0;
}

// Reference: kernels/drama.cu:793-797; src/ffi.rs:70-73.
extern "C" int dr_moe_combine(float* x, const float* Y, const int* slot_of, const float* wts, const float* sgate,
                              const float* shared, int rows, int topk, int H, cudaStream_t st) {
  if (H % 4 != 0) return -1;
  if (rows <= 0) return 0;
  pf::k_combine<<<rows, 256, 0, st>>>(x, Y, slot_of, wts, sgate, shared, topk, H);
  return 0;
}

// act: scratch of 16 bits per (slot, j); this implementation keeps the SwiGLU intermediate there as fp16.
// Reference: kernels/drama.cu:961-968; src/ffi.rs:61-64. H = 2048 and I = 512 only, else -1.
extern "C" int dr_moe_prefill(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                              const __nv_bfloat16* xp, const int* offsets, const int* counts, __nv_bfloat16* act, float* y,
                              int E, int H, int I, cudaStream_t st) {
  if (H != pf::H || I != pf::I) return -1;
  if (E <= 0) return 0;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (dev.prefill_mma) {
    // tensor-core path: two persistent grouped GEMMs (moe_prefill_mma.cuh)
    drb_launch(pfmma::k_grouped<0, 0>, dim3(pfmma::BLOCKS_PER_SM * dev.sms), dim3(pfmma::THREADS), pfmma::SMEM_BYTES, st, false, gu_q, (const void*)gu_sm,
               (const void*)xp, (void*)act, offsets, counts, E);
    drb_launch(pfmma::k_grouped<1, 0>, dim3(pfmma::BLOCKS_PER_SM * dev.sms), dim3(pfmma::THREADS), pfmma::SMEM_BYTES, st, false, d_q, (const void*)d_sm,
               (const void*)act, (void*)y, offsets, counts, E);
    return 0;
  }
  pf::k_pf_gate_up<<<dim3(E, I / 16), 256, 0, st>>>(gu_q, gu_sm, xp, offsets, counts, reinterpret_cast<__half*>(act));
  pf::k_pf_down<<<dim3(E, H / 32), 256, 0, st>>>(d_q, d_sm, reinterpret_cast<const __half*>(act), offsets, counts, y);
  return 0;
}

// The same grouped GEMMs over block-FP8 experts (layouts as dr_moe_decode_fp8). Tensor-core path only: there is no
// CUDA-core variant of it, so DRB_PREFILL=simt makes this call return -1.
// Reference: kernels/drama.cu:971-1109; src/ffi.rs:52-55. H = 2048 and I = 512 only, else -1.
extern "C" int dr_moe_prefill_fp8(const uint8_t* gu_w, const float* gu_s, const uint8_t* d_w, const float* d_s,
                                  const __nv_bfloat16* xp, const int* offsets, const int* counts, __nv_bfloat16* act, float* y,
                                  int E, int H, int I, cudaStream_t st) {
  if (H != pf::H || I != pf::I) return -1;
  if (E <= 0) return 0;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (!dev.prefill_mma) return -1;
  drb_launch(pfmma::k_grouped<0, 1>, dim3(pfmma::BLOCKS_PER_SM * dev.sms), dim3(pfmma::THREADS), pfmma::SMEM_BYTES, st, false, gu_w, (const void*)gu_s,
             (const void*)xp, (void*)act, offsets, counts, E);
  drb_launch(pfmma::k_grouped<1, 1>, dim3(pfmma::BLOCKS_PER_SM * dev.sms), dim3(pfmma::THREADS), pfmma::SMEM_BYTES, st, false, d_w, (const void*)d_s,
             (const void*)act, (void*)y, offsets, counts, E);
  return 0;
}

// Reference: kernels/drama.cu:1130-1134; src/ffi.rs:74. K a multiple of 128.
extern "C" int dr_dequant_q8(const int8_t* W, const __half* S, __nv_bfloat16* out, int N, int K, cudaStream_t st) {
  if (K % 128 != 0) return -1;
  const size_t n = (size_t)N * K;
  if (n == 0) return 0;
  pf::k_dequant_q8<<<(unsigned)((n / 16 + 255) / 256), 256, 0, st>>>(W, S, out, n, K);
  return 0;
}

// Reference: kernels/drama.cu:1163-1166; src/ffi.rs:75.
extern "C" int dr_f32_to_bf16(const float* x, __nv_bfloat16* y, size_t n, cudaStream_t st) {
  if (n == 0) return 0;
  pf::k_f32_to_bf16<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, y, n);
  return 0;
}

// Reference: kernels/drama.cu:1176-1180; src/ffi.rs:76.
extern "C" int dr_swiglu_rows(const float* h, __nv_bfloat16* y, int rows, int I, cudaStream_t st) {
  const size_t n = (size_t)rows * I;
  if (n == 0) return 0;
  pf::k_swiglu_rows<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(h, y, rows, I);
  return 0;
}

// Reference: kernels/drama.cu:1198-1202; src/ffi.rs:77.
extern "C" int dr_rmsnorm(const float* x, const float* w, float* y, __nv_bfloat16* yb, int rows, int D, float eps,
                          cudaStream_t st) {
  if (rows <= 0) return 0;
  pf::k_rmsnorm<<<rows, 256, 0, st>>>(x, w, y, yb, D, eps);
  return 0;
}
