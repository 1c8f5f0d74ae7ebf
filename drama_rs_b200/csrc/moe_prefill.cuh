// Prefill-side kernels of the MoE path: per-row routing bookkeeping (count / permute / combine and the fused
// grouping step), the launchers of the expert-grouped GEMMs (moe_prefill_mma.cuh), and the elementwise helpers the
// reference's prefill calls around cuBLAS (dequant_q8, f32_to_bf16, swiglu_rows, rmsnorm).
//
// Replaces kernels/drama.cu:744-968 and 1114-1202 of the reference, same C signatures
// (src/ffi.rs:61-77).
#pragma once

#include "common.cuh"

namespace pf {

constexpr int H = 2048, I = 512;

// ------------------------------------------------------------------------------------------
// bookkeeping

// Histogram of the chosen experts. Each block counts its 1024 pairs in shared memory and adds only its non-empty
// bins to the global counts: a few hundred global atomics per block instead of one per pair on a handful of hot
// addresses (with Zipf routing a fifth of all pairs name the same expert).
constexpr int CNT_BINS = 1024;
__global__ void __launch_bounds__(256) k_count(const int* __restrict__ idx, int n, int* __restrict__ counts) {
  pdl_wait();
  __shared__ int bins[CNT_BINS];
  for (int i = threadIdx.x; i < CNT_BINS; i += blockDim.x) bins[i] = 0;
  __syncthreads();
  const int base = blockIdx.x * 1024;
  int big[4], nbig = 0;  // experts beyond the shared bins go straight to global memory
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = base + j * 256 + threadIdx.x;
    if (i < n) {
      const int e = __ldg(idx + i);
      if (e < CNT_BINS) atomicAdd(&bins[e], 1);
      else big[nbig++] = e;
    }
  }
  for (int j = 0; j < nbig; ++j) atomicAdd(counts + big[j], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < CNT_BINS; i += blockDim.x)
    if (bins[i]) atomicAdd(counts + i, bins[i]);
}

// One warp per (row, k) pair: lane 0 claims the next slot of the pair's expert, the warp copies the row with
// 16-byte accesses. Eight pairs per block.
__global__ void __launch_bounds__(256)
    k_permute(const int* __restrict__ idx, int pairs, int topk, const int* __restrict__ offsets, int* __restrict__ fill,
              int* __restrict__ slot_of, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ xp, int Hd) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i >= pairs) return;
  int slot = 0;
  if (lane == 0) {
    const int e = __ldg(idx + i);
    slot = __ldg(offsets + e) + atomicAdd(fill + e, 1);
    slot_of[i] = slot;
  }
  slot = __shfl_sync(0xffffffffu, slot, 0);
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / topk) * Hd);
  uint4* dst = reinterpret_cast<uint4*>(xp + (size_t)slot * Hd);
  for (int c = lane; c < Hd / 8; c += 32) dst[c] = __ldg(src + c);
}

// Count, scan and slot assignment in ONE launch of one block (drb_moe_group): what the reference does with a count
// kernel, a download, a host scan, an upload, a memset and the permute kernel's atomics (src/engine.rs:565-580).
// counts[e], offsets[e] (exclusive scan), slot_of[pair] = offsets[e] + rank of the pair among its expert's pairs,
// row_of[slot] = pair / topk. The grouped GEMM reads its operand rows through row_of, so no permuted copy of the
// rows is ever written. e_lo / e_n restrict the grouping to experts [e_lo, e_lo + e_n) (an expert-parallel rank's
// slice; pairs of other experts get slot -1); local expert ids are e - e_lo.
constexpr int GRP_THREADS = 1024, GRP_MAX_E = 1024;
// With cap > 0 the pairs are what an expert-parallel rank received: `world` blocks of blk_rows rows of row_ints
// 32-bit words each; block b holds cap row slots followed by the cap expert ids of those rows (one int each, the
// region padded to whole rows). Pair j = (block j / cap, slot j % cap); its id is read from the block's id region,
// row_of[slot] is the row's index in the buffer (in rows), pair_of[slot] = j. cap = 0: idx is a plain array,
// row_of[slot] = pair / topk, pair_of is not written.
__global__ void __launch_bounds__(GRP_THREADS)
    k_group(const int* __restrict__ idx, int pairs, int topk, int e_lo, int e_n, int* __restrict__ counts,
            int* __restrict__ offsets, int* __restrict__ slot_of, int* __restrict__ row_of, int* __restrict__ pair_of,
            int cap, int blk_rows, int row_ints) {
  pdl_wait();
  __shared__ int cnt[GRP_MAX_E];
  __shared__ int offs[GRP_MAX_E];
  __shared__ int warp_tot[GRP_THREADS / 32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  auto expert_of = [&](int p) {
    if (cap <= 0) return __ldg(idx + p);
    const int b = p / cap, i = p - b * cap;
    return __ldcg(idx + ((size_t)b * blk_rows + cap) * row_ints + i);
  };
  for (int i = t; i < e_n; i += GRP_THREADS) cnt[i] = 0;
  __syncthreads();
  // rank of every pair among its expert's pairs (the order inside an expert is arbitrary: every slot is computed
  // independently and the combine step sums in a fixed order)
  for (int p = t; p < pairs; p += GRP_THREADS) {
    const int e = expert_of(p) - e_lo;
    slot_of[p] = (e >= 0 && e < e_n) ? atomicAdd(&cnt[e], 1) : -1;
  }
  __syncthreads();
  // exclusive scan of the counts: one value per thread (e_n <= 1024)
  const int c = t < e_n ? cnt[t] : 0;
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_tot[lane], in2 = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, in2, o);
      if (lane >= o) in2 += u;
    }
    warp_tot[lane] = in2 - v;  // exclusive over the warps
  }
  __syncthreads();
  if (t < e_n) {
    const int o = warp_tot[warp] + incl - c;
    offs[t] = o;
    counts[t] = c;
    offsets[t] = o;
  }
  __syncthreads();
  for (int p = t; p < pairs; p += GRP_THREADS) {
    const int e = expert_of(p) - e_lo;
    if (e >= 0 && e < e_n) {
      const int slot = offs[e] + slot_of[p];
      slot_of[p] = slot;
      if (cap <= 0) {
        row_of[slot] = p / topk;
      } else {
        const int b = p / cap;
        row_of[slot] = b * blk_rows + (p - b * cap);
        pair_of[slot] = p;
      }
    }
  }
}

// Expert-parallel dispatch, sender side, step 1 (one block): every (row, k) pair gets a slot in the block of the rank
// that owns its expert. send is `world` blocks of blk_rows rows of row_ints words (layout as in k_group); the pair's
// local expert id goes to the block's id region, unused slots get the id `per` (one past the owner's last expert:
// the owner's grouping skips them). slot_of[pair] = owner * cap + slot (what the combine step indexes the returned
// results with), dst_row[pair] = the row of `send` that the pair's row must be copied to (-1: dropped).
// A pair that finds its block full is dropped, its slot_of points at a valid slot of the block, and *overflow is set:
// the step's result is then void and the caller must repeat it with a larger capacity. Nothing waits or faults.
// With `peers` (device array of every rank's receive buffer) block o is not a part of `send` but this rank's slot in
// peer o's receive buffer: the ids and rows are stored straight into the owner's memory over NVLink, and every
// thread fences at system scope after its stores (the flag that announces them is written by a later kernel).
__global__ void __launch_bounds__(GRP_THREADS)
    k_ep_plan(const int* __restrict__ idx, int pairs, int per, int world, int cap, int blk_rows, int row_ints,
              int* __restrict__ send_local, int* __restrict__ slot_of, int* __restrict__ dst_row, unsigned* __restrict__ overflow,
              int* const* __restrict__ peers, int rank) {
  pdl_wait();
  __shared__ int cnt[64];
  __shared__ int* blk[64];
  const int t = threadIdx.x;
  if (t < 64) cnt[t] = 0;
  if (t < world) blk[t] = peers ? peers[t] + (size_t)rank * blk_rows * row_ints : send_local + (size_t)t * blk_rows * row_ints;
  __syncthreads();
  for (int p = t; p < pairs; p += GRP_THREADS) {
    const int e = __ldg(idx + p);
    const int o = e / per;
    const int r = atomicAdd(&cnt[o], 1);
    if (r < cap) {
      blk[o][(size_t)cap * row_ints + r] = e - o * per;
      slot_of[p] = o * cap + r;
      dst_row[p] = o * blk_rows + r;
    } else {
      atomicExch(overflow, 1u);
      slot_of[p] = o * cap;
      dst_row[p] = -1;
    }
  }
  __syncthreads();
  for (int j = t; j < world * cap; j += GRP_THREADS) {
    const int o = j / cap, r = j - o * cap;
    if (r >= cnt[o]) blk[o][(size_t)cap * row_ints + r] = per;
  }
  if (peers) __threadfence_system();
}

// Step 2: one warp per pair copies its row (row_bytes each, 16-byte accesses) to its place in the send buffer.
__global__ void __launch_bounds__(256)
    k_ep_scatter(const unsigned char* __restrict__ rows, int pairs, int topk, const int* __restrict__ dst_row,
                 unsigned char* __restrict__ send, int row_bytes, unsigned char* const* __restrict__ peers, int rank, int blk_rows) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= pairs) return;
  const int d = __ldg(dst_row + p);
  if (d < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(rows + (size_t)(p / topk) * row_bytes);
  uint4* dst;
  if (peers) {
    const int o = d / blk_rows;
    dst = reinterpret_cast<uint4*>(peers[o] + ((size_t)rank * blk_rows + (d - o * blk_rows)) * row_bytes);
  } else {
    dst = reinterpret_cast<uint4*>(send + (size_t)d * row_bytes);
  }
  for (int c = lane; c < row_bytes / 16; c += 32) dst[c] = __ldg(src + c);
  if (peers) __threadfence_system();
}

// The exchange of an expert-parallel step over NVLink peer stores (drb_ep_put / drb_ep_signal / drb_ep_wait): block p of
// this rank's send buffer goes straight into peer p's receive buffer, slot `rank`, with 16-byte stores; every
// writing thread fences at system scope after its stores, so that the flag the next kernel writes to the peer
// can only be seen after the data.
__global__ void __launch_bounds__(256)
    k_ep_put(const uint4* __restrict__ send, uint4* const* __restrict__ peer_recv, int rank, size_t block_vecs) {
  pdl_wait();
  const int p = blockIdx.y;
  const uint4* src = send + (size_t)p * block_vecs;
  uint4* dst = peer_recv[p] + (size_t)rank * block_vecs;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < block_vecs; i += (size_t)gridDim.x * blockDim.x) dst[i] = __ldg(src + i);
  __threadfence_system();
}

// ++*step; then peer p's flag word `rank` takes the new step number (one thread per peer).
__global__ void __launch_bounds__(64) k_ep_signal(unsigned* const* __restrict__ peer_flags, int world, int rank, unsigned* __restrict__ step) {
  pdl_wait();
  __shared__ unsigned now;
  if (threadIdx.x == 0) now = ++*step;
  __syncthreads();
  __threadfence_system();
  if ((int)threadIdx.x < world) {
    volatile unsigned* f = peer_flags[threadIdx.x] + rank;
    *f = now;
  }
}

// ++*step; then waits until every peer's flag has reached the new step number. Bounded: a peer that never signals
// costs `limit` polls, sets the error word and lets the step run on (its result is void).
__global__ void __launch_bounds__(64) k_ep_wait(const unsigned* __restrict__ flags, int world, unsigned* __restrict__ step, unsigned limit) {
  pdl_wait();
  __shared__ unsigned now;
  if (threadIdx.x == 0) now = ++*step;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const volatile unsigned* f = flags + threadIdx.x;
    unsigned it = 0;
    // signed distance: the counters wrap together
    while ((int)(*f - now) < 0) {
      if (++it >= limit) {
        atomicMax(&g_drb_error, (unsigned)DRB_ERR_GRID_WAIT);
        break;
      }
      if (it > 64) __nanosleep(it > 4096 ? 256 : 32);
    }
  }
  __threadfence_system();
}

// k_ep_signal and k_ep_wait in one launch: announce this rank's stores to every peer, then wait for every peer's.
__global__ void __launch_bounds__(64)
    k_ep_sync(unsigned* const* __restrict__ peer_flags, const unsigned* __restrict__ flags, int world, int rank, unsigned* __restrict__ steps,
              unsigned limit) {
  pdl_wait();
  __shared__ unsigned now_s, now_w;
  if (threadIdx.x == 0) now_s = ++steps[0], now_w = ++steps[1];
  __syncthreads();
  __threadfence_system();
  if ((int)threadIdx.x < world) {
    volatile unsigned* out = peer_flags[threadIdx.x] + rank;
    *out = now_s;
    const volatile unsigned* f = flags + threadIdx.x;
    unsigned it = 0;
    while ((int)(*f - now_w) < 0) {
      if (++it >= limit) {
        atomicMax(&g_drb_error, (unsigned)DRB_ERR_GRID_WAIT);
        break;
      }
      if (it > 64) __nanosleep(it > 4096 ? 256 : 32);
    }
  }
  __threadfence_system();
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

// Row-wise RMSNorm ("+1" already folded into w). Writes f32 and/or a 16-bit copy: bf16, or (F16) fp16 clamped to its range.
template <bool F16>
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
    if (yb) {
      if (F16) reinterpret_cast<__half*>(yb)[(size_t)blockIdx.x * D + i] = pfmma::f2h_sat(v);
      else yb[(size_t)blockIdx.x * D + i] = __float2bfloat16(v);
    }
  }
}

// Router logits whose value for a row does not depend on how many rows are computed together: every (row, output)
// pair is one warp's dot product in a fixed order (lane l takes the 16-byte chunks l, l + 32, ... of the K = 2048
// inputs, products exact in fp32, one fixed butterfly). A library GEMM picks its kernel by the batch size (measured:
// logits of the same row differ by 1.2e-6 between a batch of 300 and a batch of 38), which would let the routing of
// a row depend on how the rows are spread over the GPUs. Block (x, y) = RB rows x the outputs y, y + gridDim.y, ...;
// its warp w takes every 8th of those. The split over y only adds parallelism: it does not change any sum.
// F16: the rows are fp16 instead of bf16 (the weights are bf16 either way).
constexpr int RL_RB = 4, RL_K = 2048, RL_SPLIT = 9;
template <bool F16>
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
          float x0, x1;
          if (F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw[t]));
            x0 = f.x, x1 = f.y;
          } else {
            x0 = __uint_as_float(xw[t] << 16), x1 = __uint_as_float(xw[t] & 0xffff0000u);
          }
          acc[r] = fmaf(__uint_as_float(ww[t] << 16), x0, acc[r]);
          acc[r] = fmaf(__uint_as_float(ww[t] & 0xffff0000u), x1, acc[r]);
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
  if ((e = drb_carveout(k_router_logits<false>)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_router_logits<true>)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_count)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_permute)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_combine)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_group)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_ep_plan)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_ep_scatter)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_ep_put)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_dequant_q8)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_f32_to_bf16)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_swiglu_rows)) != cudaSuccess) return e;
  if ((e = drb_carveout(k_rmsnorm<true>)) != cudaSuccess) return e;
  return drb_carveout(k_rmsnorm<false>);
}

}  // namespace pf

// Reference: kernels/drama.cu:750-753; src/ffi.rs:65. counts must be zeroed by the caller.
extern "C" int dr_moe_count(const int* idx, int n, int* counts, cudaStream_t st) {
  if (n <= 0) return 0;
  pf::k_count<<<(n + 1023) / 1024, 256, 0, st>>>(idx, n, counts);
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
  pf::k_router_logits<false><<<dim3((rows + pf::RL_RB - 1) / pf::RL_RB, pf::RL_SPLIT), 256, 0, st>>>(xb, w, logits, rows, e1, beta);
  return 0;
}

// The two calls above for rows kept in fp16 (no counterpart in the reference, whose prefill rounds the normalised rows
// to bf16: src/engine.rs:499): drb_rmsnorm_f16 writes the normalised rows as fp16 (clamped to +-65504),
// drb_router_logits_f16 reads them. With drb_moe_prefill_block(x_f16 = 1) the whole block then works on rows with
// eleven significant bits instead of eight.
extern "C" int drb_rmsnorm_f16(const float* x, const float* w, __half* yh, int rows, int D, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  pf::k_rmsnorm<true><<<rows, 256, 0, st>>>(x, w, nullptr, reinterpret_cast<__nv_bfloat16*>(yh), D, eps);
  return 0;
}
extern "C" int drb_router_logits_f16(const __half* xh, const __nv_bfloat16* w, float* logits, int rows, int e1, int h, float beta,
                                     cudaStream_t st) {
  if (h != pf::RL_K) return -1;
  if (rows <= 0 || e1 <= 0) return 0;
  pf::k_router_logits<true><<<dim3((rows + pf::RL_RB - 1) / pf::RL_RB, pf::RL_SPLIT), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(xh), w, logits, rows, e1, beta);
  return 0;
}

// Reference: kernels/drama.cu:774-778; src/ffi.rs:66-69. fill must be zeroed by the caller.
extern "C" int dr_moe_permute(const int* idx, int rows, int topk, const int* offsets, int* fill, int* slot_of,
                              const __nv_bfloat16* x, __nv_bfloat16* xp, int H, cudaStream_t st) {
  if (H % 8 != 0) return -1;
  if (rows * topk <= 0) return 0;
  pf::k_permute<<<(rows * topk + 7) / 8, 256, 0, st>>>(idx, rows * topk, topk, offsets, fill, slot_of, x, xp, H);
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

// act: scratch of 16 bits per (slot, j); this implementation keeps the SwiGLU intermediate there as fp16
// (values beyond +-65504 are clamped to that range).
// Reference: kernels/drama.cu:961-968; src/ffi.rs:61-64. H = 2048 and I = 512 only, else -1.
extern "C" int dr_moe_prefill(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                              const __nv_bfloat16* xp, const int* offsets, const int* counts, __nv_bfloat16* act, float* y,
                              int E, int H, int I, cudaStream_t st) {
  if (H != pf::H || I != pf::I) return -1;
  if (E <= 0) return 0;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  const dim3 grid(pfmma::BLOCKS_PER_SM * dev.sms), block(pfmma::THREADS);
  drb_launch(pfmma::k_grouped<0, 0, false>, grid, block, pfmma::SMEM_BYTES, st, false, gu_q, (const void*)gu_sm, (const void*)xp,
             (void*)act, offsets, counts, E, pfmma::SharedExpert{}, (const int*)nullptr, 0, (const int*)nullptr);
  drb_launch(pfmma::k_grouped<1, 0, false>, grid, block, pfmma::SMEM_BYTES, st, false, d_q, (const void*)d_sm, (const void*)act,
             (void*)y, offsets, counts, E, pfmma::SharedExpert{}, (const int*)nullptr, 0, (const int*)nullptr);
  return 0;
}

// No counterpart in the reference. Count, exclusive scan and slot assignment of the (row, k) pairs in one launch:
// counts[e_n], offsets[e_n], slot_of[rows * topk] (-1 for pairs whose expert lies outside [e_lo, e_lo + e_n)),
// row_of[slot] = row. Replaces dr_moe_count + the host scan + dr_moe_permute of src/engine.rs:565-580 when the
// grouped GEMM is drb_moe_prefill_block, which reads its rows through row_of. e_n <= 1024, else -1.
extern "C" int drb_moe_group(const int* idx, int rows, int topk, int e_lo, int e_n, int* counts, int* offsets, int* slot_of,
                             int* row_of, cudaStream_t st) {
  if (e_n <= 0 || e_n > pf::GRP_MAX_E || topk <= 0) return -1;
  drb_launch(pf::k_group, dim3(1), dim3(pf::GRP_THREADS), 0, st, false, idx, rows * topk, topk, e_lo, e_n, counts, offsets,
             slot_of, row_of, (int*)nullptr, 0, 0, 0);
  return 0;
}

// Expert parallelism (no counterpart in the reference, which is single-GPU). Rows travel between ranks in a buffer of
// `world` blocks; a block is blk_rows = cap + ceil(4 cap / row_bytes) rows of row_bytes bytes: cap row slots, then the
// cap local expert ids of those rows (int32), padded to whole rows. One collective moves rows and ids together.
//   drb_ep_pack    sender: places this rank's (row, k) pairs (idx [rows, topk], experts per rank `per`) into `send`,
//                  slot_of [rows * topk] = owner * cap + slot for the combine step, dst_row [rows * topk] scratch.
//                  *overflow (device word, zeroed by the caller) is set when a block was full: the result is void then.
//   drb_ep_group   owner: groups the received world * cap pairs by local expert: counts / offsets [per],
//                  slot_of [world * cap] scratch, row_of [slot] = row of `recv` (operand gather of the grouped GEMM),
//                  pair_of [slot] = position of the pair in receive order (where the result row goes).
// row_bytes % 16 == 0, world <= 64, per <= 1024; -1 otherwise.
extern "C" int drb_ep_block_rows(int cap, int row_bytes) { return cap + (4 * cap + row_bytes - 1) / row_bytes; }
extern "C" int drb_ep_pack(const void* rows, const int* idx, int n_rows, int topk, int per, int world, int cap, int row_bytes,
                           void* send, int* slot_of, int* dst_row, unsigned* overflow, cudaStream_t st) {
  if (row_bytes % 16 != 0 || world <= 0 || world > 64 || per <= 0 || cap <= 0 || topk <= 0) return -1;
  const int pairs = n_rows * topk;
  const int blk_rows = drb_ep_block_rows(cap, row_bytes);
  drb_launch(pf::k_ep_plan, dim3(1), dim3(pf::GRP_THREADS), 0, st, false, idx, pairs, per, world, cap, blk_rows, row_bytes / 4,
             (int*)send, slot_of, dst_row, overflow, (int* const*)nullptr, 0);
  if (pairs > 0)
    drb_launch(pf::k_ep_scatter, dim3((pairs + 7) / 8), dim3(256), 0, st, false, (const unsigned char*)rows, pairs, topk,
               (const int*)dst_row, (unsigned char*)send, row_bytes, (unsigned char* const*)nullptr, 0, blk_rows);
  return 0;
}
// drb_ep_pack with the blocks stored straight into the owners' receive buffers (peer_recv: device array of `world`
// pointers as for drb_ep_put; this rank's block in peer o's buffer is block `rank`). Follow with drb_ep_signal.
extern "C" int drb_ep_pack_peers(const void* rows, const int* idx, int n_rows, int topk, int per, int world, int cap, int row_bytes,
                                 void* const* peer_recv, int rank, int* slot_of, int* dst_row, unsigned* overflow, cudaStream_t st) {
  if (row_bytes % 16 != 0 || world <= 0 || world > 64 || per <= 0 || cap <= 0 || topk <= 0 || !peer_recv || rank < 0 || rank >= world)
    return -1;
  const int pairs = n_rows * topk;
  const int blk_rows = drb_ep_block_rows(cap, row_bytes);
  drb_launch(pf::k_ep_plan, dim3(1), dim3(pf::GRP_THREADS), 0, st, false, idx, pairs, per, world, cap, blk_rows, row_bytes / 4,
             (int*)nullptr, slot_of, dst_row, overflow, reinterpret_cast<int* const*>(peer_recv), rank);
  if (pairs > 0)
    drb_launch(pf::k_ep_scatter, dim3((pairs + 7) / 8), dim3(256), 0, st, false, (const unsigned char*)rows, pairs, topk,
               (const int*)dst_row, (unsigned char*)nullptr, row_bytes, reinterpret_cast<unsigned char* const*>(peer_recv), rank, blk_rows);
  return 0;
}
extern "C" int drb_ep_group(const void* recv, int world, int cap, int row_bytes, int per, int* counts, int* offsets, int* slot_of,
                            int* row_of, int* pair_of, cudaStream_t st) {
  if (row_bytes % 16 != 0 || world <= 0 || per <= 0 || per > pf::GRP_MAX_E || cap <= 0) return -1;
  drb_launch(pf::k_group, dim3(1), dim3(pf::GRP_THREADS), 0, st, false, (const int*)recv, world * cap, 1, 0, per, counts, offsets,
             slot_of, row_of, pair_of, cap, drb_ep_block_rows(cap, row_bytes), row_bytes / 4);
  return 0;
}

// The expert-parallel exchange over NVLink peer stores instead of a library collective (no counterpart in the
// reference). peer_recv / peer_flags: device arrays of `world` pointers, entry p = rank p's receive buffer / flag
// array (memory every rank can store to: symmetric memory), this rank's own included.
//   drb_ep_put     block p (block_bytes each) of `send` -> peer p's receive buffer at slot `rank`
//   drb_ep_signal  ++*step (device word, zero at start on every rank); peer p's flag [rank] = *step
//   drb_ep_wait    ++*step (another device word, zero at start); returns once flags [0, world) have all reached it, or
//                  after poll_limit polls (error word set, the step's result is void)
// One exchange = put, signal on the sender; wait on the receiver before it reads. A rank starts the next exchange
// into a peer's buffer only after that peer's reply to the current one, so a buffer is never overwritten while it
// is read. block_bytes % 16 == 0, world <= 64, else -1.
extern "C" int drb_ep_put(const void* send, void* const* peer_recv, int world, int rank, size_t block_bytes, cudaStream_t st) {
  if (!send || !peer_recv || world <= 0 || world > 64 || rank < 0 || rank >= world || block_bytes % 16 != 0) return -1;
  if (block_bytes == 0) return 0;
  const size_t vecs = block_bytes / 16;
  const unsigned per = (unsigned)((vecs + 4095) / 4096);  // about sixteen 16-byte stores per thread
  drb_launch(pf::k_ep_put, dim3(per < 1 ? 1 : (per > 64 ? 64 : per), (unsigned)world), dim3(256), 0, st, false,
             static_cast<const uint4*>(send), reinterpret_cast<uint4* const*>(peer_recv), rank, vecs);
  return 0;
}
extern "C" int drb_ep_signal(unsigned* const* peer_flags, int world, int rank, unsigned* step, cudaStream_t st) {
  if (!peer_flags || !step || world <= 0 || world > 64 || rank < 0 || rank >= world) return -1;
  drb_launch(pf::k_ep_signal, dim3(1), dim3(64), 0, st, false, peer_flags, world, rank, step);
  return 0;
}
// drb_ep_signal followed by drb_ep_wait in one launch; steps: two device words (signalled, awaited), zero at start.
extern "C" int drb_ep_sync(unsigned* const* peer_flags, const unsigned* flags, int world, int rank, unsigned* steps, unsigned poll_limit,
                           cudaStream_t st) {
  if (!peer_flags || !flags || !steps || world <= 0 || world > 64 || rank < 0 || rank >= world || poll_limit == 0) return -1;
  drb_launch(pf::k_ep_sync, dim3(1), dim3(64), 0, st, false, peer_flags, flags, world, rank, steps, poll_limit);
  return 0;
}
extern "C" int drb_ep_wait(const unsigned* flags, int world, unsigned* step, unsigned poll_limit, cudaStream_t st) {
  if (!flags || !step || world <= 0 || world > 64 || poll_limit == 0) return -1;
  drb_launch(pf::k_ep_wait, dim3(1), dim3(64), 0, st, false, flags, world, step, poll_limit);
  return 0;
}

// drb_moe_prefill_block and drb_moe_prefill_block_peers (no counterpart in the reference). The routed experts AND the
// int8 shared expert of one prefill block in two launches: dr_moe_prefill with (a) the operand rows read in place through row_of (xb holds the normalised rows in row
// order, [rows, H], bf16 or with x_f16 != 0 fp16; nothing is permuted) and (b) the shared expert as one more expert that owns every row, its
// int8 weights dequantised into the same tensor-core tiles (sh_act: fp16 scratch [rows, I]; sh_out: f32 [rows, H]).
// The reference runs the shared expert through cuBLAS on weights dequantised to bf16 (src/engine.rs:351-355, 560-562);
// here no library GEMM and no bf16 copy of the weights is involved. rows_sh = 0 skips the shared expert, E = 0 the
// routed ones. y_row_of (or NULL): slot -> row of y for the routed results. Limits as dr_moe_prefill.
// Every pointer of a part that runs must be a valid device address; with E = 0 or rows_sh = 0 the arrays of the part
// that does not run are not used, but must still be valid addresses (any buffer will do, NULL will not): the compiler
// may issue a load ahead of the branch that decides whether its value is needed. row_of and y_row_of may be NULL.
// fp16 rows and E <= 256 take the kernels of moe_prefill_tma.cuh (and only they can store results to peers: peer_y);
// bf16 rows, or more experts, the kernels of moe_prefill_mma.cuh.
static int prefill_block_impl(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                                     const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                                     const __nv_bfloat16* xb, const int* row_of, const int* offsets, const int* counts,
                                     __nv_bfloat16* act, float* y, __nv_bfloat16* sh_act, float* sh_out, int rows_sh, int E,
                                     int H, int I, int x_f16, const int* y_row_of, float* const* peer_y, int peer_cap, int peer_rank, cudaStream_t st) {
  if (H != pf::H || I != pf::I) return -1;
  if (E <= 0 && rows_sh <= 0) return 0;
  if (!gu_q || !gu_sm || !d_q || !d_sm || !sgu_q || !sgu_s || !sd_q || !sd_s || !xb || !offsets || !counts || !act || !y || !sh_act || !sh_out)
    return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  if (x_f16 && E <= pft::MAX_ITEM_SETS - 1) {
    // fp16 rows: the kernels of moe_prefill_tma.cuh (weights by tiled TMA, token tiles by asynchronous copies)
    const uint64_t ne = (uint64_t)(E > 0 ? E : 1);
    CUtensorMap m_gu, m_d, m_sgu, m_sd;
    if (pft::map_gate_up(&m_gu, gu_q, ne, I, H / 2) || pft::map_gate_up(&m_sgu, sgu_q, 1, I, H) ||
        pft::map_rows(&m_d, d_q, ne * H, I / 2) || pft::map_rows(&m_sd, sd_q, H, I))
      return -3;
    const dim3 grid2(2 * dev.sms), block2(pft::THREADS);
    const int ee = E > 0 ? E : 0, rs = rows_sh > 0 ? rows_sh : 0;
    const __half* rows16 = reinterpret_cast<const __half*>(xb);
    drb_launch(pft::k_grouped_tma<0>, grid2, block2, pft::SMEM_BYTES, st, false, m_gu, gu_sm, m_sgu, sgu_s, rows16, rows16, (void*)act,
               (void*)sh_act, offsets, counts, ee, rs, row_of, (const int*)nullptr, (float* const*)nullptr, 0, 0);
    drb_launch(pft::k_grouped_tma<1>, grid2, block2, pft::SMEM_BYTES, st, false, m_d, d_sm, m_sd, sd_s,
               reinterpret_cast<const __half*>(act), reinterpret_cast<const __half*>(sh_act), (void*)y, (void*)sh_out, offsets, counts, ee, rs,
               (const int*)nullptr, y_row_of, peer_y, peer_cap, peer_rank);
    return 0;
  }
  if (peer_y) return -1;  // results to the peers: the TMA kernels only
  const dim3 grid(pfmma::BLOCKS_PER_SM * dev.sms), block(pfmma::THREADS);
  const pfmma::SharedExpert s0{sgu_q, sgu_s, (const void*)xb, (void*)sh_act, rows_sh};
  const pfmma::SharedExpert s1{sd_q, sd_s, (const void*)sh_act, (void*)sh_out, rows_sh};
  drb_launch(pfmma::k_grouped<0, 0, true>, grid, block, pfmma::SMEM_BYTES, st, false, gu_q, (const void*)gu_sm, (const void*)xb,
             (void*)act, offsets, counts, E, s0, row_of, x_f16, (const int*)nullptr);
  drb_launch(pfmma::k_grouped<1, 0, true>, grid, block, pfmma::SMEM_BYTES, st, false, d_q, (const void*)d_sm, (const void*)act,
             (void*)y, offsets, counts, E, s1, (const int*)nullptr, 1, y_row_of);
  return 0;
}

extern "C" int drb_moe_prefill_block(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                                     const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                                     const __nv_bfloat16* xb, const int* row_of, const int* offsets, const int* counts,
                                     __nv_bfloat16* act, float* y, __nv_bfloat16* sh_act, float* sh_out, int rows_sh, int E,
                                     int H, int I, int x_f16, const int* y_row_of, cudaStream_t st) {
  return prefill_block_impl(gu_q, gu_sm, d_q, d_sm, sgu_q, sgu_s, sd_q, sd_s, xb, row_of, offsets, counts, act, y, sh_act, sh_out, rows_sh, E,
                            H, I, x_f16, y_row_of, nullptr, 0, 0, st);
}
// drb_moe_prefill_block on an expert-parallel rank, with the routed results stored straight into the home ranks'
// buffers: y_row_of[slot] = s * cap + j names the token's source rank s and its slot j in this rank's receive
// order; its result row goes to peer_y[s] (device array of every rank's result buffer [world * cap, h] f32) at row
// rank * cap + j, over NVLink, from the down GEMM's epilogue. Follow with drb_ep_signal; the home rank's
// drb_ep_wait then covers the results. fp16 rows and e <= 256 only (-1 otherwise). y is not written.
extern "C" int drb_moe_prefill_block_peers(const uint8_t* gu_q, const __half2* gu_sm, const uint8_t* d_q, const __half2* d_sm,
                                           const int8_t* sgu_q, const __half* sgu_s, const int8_t* sd_q, const __half* sd_s,
                                           const __nv_bfloat16* xb, const int* row_of, const int* offsets, const int* counts,
                                           __nv_bfloat16* act, float* y, __nv_bfloat16* sh_act, float* sh_out, int rows_sh, int E,
                                           int H, int I, const int* y_row_of, float* const* peer_y, int cap, int rank,
                                           cudaStream_t st) {
  if (!peer_y || !y_row_of || cap <= 0 || rank < 0) return -1;
  return prefill_block_impl(gu_q, gu_sm, d_q, d_sm, sgu_q, sgu_s, sd_q, sd_s, xb, row_of, offsets, counts, act, y, sh_act, sh_out, rows_sh, E,
                            H, I, 1, y_row_of, peer_y, cap, rank, st);
}

// dr_moe_prefill over block-FP8 experts (include/dramakernels.h). Reference: kernels/drama.cu:971-1109; src/ffi.rs:52-55.
extern "C" int dr_moe_prefill_fp8(const uint8_t* gu_w, const float* gu_s, const uint8_t* d_w, const float* d_s,
                                  const __nv_bfloat16* xp, const int* offsets, const int* counts, __nv_bfloat16* act, float* y,
                                  int E, int H, int I, cudaStream_t st) {
  if (H != pf::H || I != pf::I) return -1;
  if (E <= 0) return 0;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  // The weights reach the tensor cores as E4M3 (moe_prefill_fp8.cuh). DRB_FP8_DEQUANT=1 (read at every call) selects the
  // earlier kernels, whose threads turn every weight into fp16 first: the route for more than 256 experts, kept
  // selectable so that both can be compared and tested on the same inputs; same results within the parity bar.
  const char* route = getenv("DRB_FP8_DEQUANT");
  const bool dequant_route = route && route[0] == '1';
  if (!dequant_route && E <= pf8::MAX_ITEM_SETS) {
    CUtensorMap tm_gu, tm_d;
    // 256-byte L2 promotion: a chunk's box brings the next chunk's 128 bytes of every row into L2 with it
    if (pft::map_rows(&tm_gu, gu_w, (uint64_t)E * 2 * pf::I, pf::H, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) != 0) return -3;
    if (pft::map_rows(&tm_d, d_w, (uint64_t)E * pf::H, pf::I, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) != 0) return -3;
    const dim3 grid(2 * dev.sms), block(pf8::THREADS);
    // y is written last (by the down kernel); until then its first floats hold every token row's largest magnitude
    pf8::k_rowmax_bf16<<<2 * dev.sms, 256, 0, st>>>(xp, offsets, counts, E, y);
    drb_launch(pf8::k_gate_up_fp8, grid, block, pf8::SMEM, st, false, tm_gu, gu_s, xp, (const float*)y, (__half*)act, offsets, counts, E);
    drb_launch(pf8::down::k_down_fp8, grid, dim3(pf8::down::THREADS), pf8::down::SMEM, st, false, tm_d, d_s, (const __half*)act, y, offsets, counts, E);
    return 0;
  }
  const dim3 grid(pfmma::BLOCKS_PER_SM * dev.sms), block(pfmma::THREADS);
  drb_launch(pfmma::k_grouped<0, 1, false>, grid, block, pfmma::SMEM_BYTES, st, false, gu_w, (const void*)gu_s, (const void*)xp,
             (void*)act, offsets, counts, E, pfmma::SharedExpert{}, (const int*)nullptr, 0, (const int*)nullptr);
  drb_launch(pfmma::k_grouped<1, 1, false>, grid, block, pfmma::SMEM_BYTES, st, false, d_w, (const void*)d_s, (const void*)act,
             (void*)y, offsets, counts, E, pfmma::SharedExpert{}, (const int*)nullptr, 0, (const int*)nullptr);
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
  pf::k_rmsnorm<false><<<rows, 256, 0, st>>>(x, w, y, yb, D, eps);
  return 0;
}
