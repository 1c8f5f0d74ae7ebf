// Router: fused RMSNorm + bf16 router GEMV + softmax + top-k (dr_router_topk), and the
// prefill variant over precomputed logits (dr_moe_topk).
//
// Selection rule (the reference's, kernels/drama.cu:330-366 and 397-435): softmax over the E router
// logits in fp32, the k largest probabilities in descending order, ties to the lower expert index,
// weights divided by their sum accumulated in rank order; logit E is the shared-expert gate.
//
// The top-k is done by rank counting instead of k serial arg-max rounds: every warp ranks its 32
// probabilities against each other with shuffles, the at most 8*topk survivors are ranked against
// each other through shared memory, and the entries whose final rank is below k write themselves
// to their slot. Two block barriers instead of two per selected expert.
#pragma once

#include "common.cuh"

namespace router {

constexpr int THREADS = 256;  // one probability per thread in the tail: E <= 256
constexpr int MAX_TOPK = 32;

// a ranks before b: larger probability, or equal probability and lower index.
DRB_DEV bool before(float pa, int ia, float pb, int ib) { return pa > pb || (pa == pb && ia < ib); }

struct TopkSmem {
  float red[32];
  unsigned ck[8 * MAX_TOPK];
  int ci[8 * MAX_TOPK];
  float top[MAX_TOPK];
  int ncand[8];
};

// Sum over a 256-thread block with the reference's tree: xor-butterfly inside each warp, then the
// same butterfly over the eight warp totals (kernels/drama.cu:39-47). Every thread gets the total.
DRB_DEV float block_sum_256(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  return warp_sum(lane < 8 ? red[lane] : 0.f);
}

DRB_DEV float block_max_256(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  return warp_max(lane < 8 ? red[lane] : -INFINITY);
}

// Softmax + top-k of one row of logits by a 256-thread block. Thread e holds logit e (or -inf).
//
// Selection in two levels. Every warp extracts the best min(topk, 32) of its 32 probabilities by
// repeated warp arg-max (the lowest lane among equal values wins, and lane order is index order).
// Warp 0 then merges the eight sorted lists: lane w holds the head of warp w's list, and among
// equal heads the lowest lane again holds the lowest expert index.
DRB_DEV void softmax_topk(float v, int E, int topk, int* __restrict__ idx, float* __restrict__ wts, TopkSmem& sm) {
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const float m = block_max_256(v, sm.red);
  const float ex = e < E ? expf(v - m) : 0.f;
  const float z = block_sum_256(ex, sm.red);
  const float p = e < E ? ex / z : -1.f;
  // Probabilities are >= 0, so their bit patterns order like unsigned integers and one redux
  // instruction finds a warp's maximum; spent or invalid entries are 0 and an all-zero round marks the end.
  const int kk = topk < 32 ? topk : 32;
  unsigned mine = e < E ? __float_as_uint(p) + 1u : 0u;  // + 1: a valid probability of exactly 0 still beats "spent"
  for (int r = 0; r < kk; ++r) {
    const unsigned best = __reduce_max_sync(0xffffffffu, mine);
    const int src = __ffs(__ballot_sync(0xffffffffu, mine == best)) - 1;
    if (lane == r) {
      sm.ck[warp * MAX_TOPK + r] = best;
      sm.ci[warp * MAX_TOPK + r] = (warp << 5) + src;
    }
    if (lane == src) mine = 0u;
  }
  __syncthreads();
  if (warp != 0) return;
  int head = 0;
  unsigned hk = lane < 8 ? sm.ck[lane * MAX_TOPK] : 0u;
  float my_top = 0.f;
  for (int r = 0; r < topk; ++r) {
    const unsigned best = __reduce_max_sync(0xffffffffu, hk);
    const int src = __ffs(__ballot_sync(0xffffffffu, hk == best)) - 1;
    const int win = __shfl_sync(0xffffffffu, lane < 8 ? sm.ci[lane * MAX_TOPK + head] : 0, src);
    if (lane == r) {
      my_top = __uint_as_float(best - 1u);
      idx[r] = win;
    }
    if (lane == src) {
      ++head;
      hk = head < kk ? sm.ck[lane * MAX_TOPK + head] : 0u;
    }
  }
  float total = 0.f;
  for (int r = 0; r < topk; ++r) total += __shfl_sync(0xffffffffu, my_top, r);  // rank order, as the reference accumulates
  if (lane < topk) wts[lane] = my_top / total;
}

// grid = rows of logits; logits has E + 1 valid columns per row at the given stride.
__global__ void __launch_bounds__(THREADS)
    k_moe_topk(const float* __restrict__ logits, int E, int topk, int stride, int* __restrict__ idx,
               float* __restrict__ wts, float* __restrict__ sgate) {
  __shared__ TopkSmem sm;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* l = logits + (size_t)r * stride;
  const float v = (int)threadIdx.x < E ? l[threadIdx.x] : -INFINITY;
  softmax_topk(v, E, topk, idx + (size_t)r * topk, wts + (size_t)r * topk, sm);
  if (threadIdx.x == 0) sgate[r] = l[E];
}

// Decode router. Block b owns rows [b*R, b*R + R) of the [E+1, 2048] bf16 matrix, fetched with one
// bulk copy issued before the dependency wait. After the wait every block normalises x itself,
// computes its logits, and the last block to arrive (atomic counter, left at zero) runs the tail.
constexpr int K = 2048;
constexpr int ROWS_PER_BLOCK = 2;

struct Smem {
  __align__(16) unsigned char w[ROWS_PER_BLOCK * K * 2];
  uint64_t full;
  float part[ROWS_PER_BLOCK][8];
  float red[32];
  float inv_rms;
  int last;
  TopkSmem tk;
};

__global__ void __launch_bounds__(THREADS)
    k_router_topk(const __nv_bfloat16* __restrict__ W, const float* __restrict__ x, const float* __restrict__ nw, float eps,
                  float* logits, int E, int topk, int* __restrict__ idx, float* __restrict__ wts,
                  float* __restrict__ sgate, unsigned* counter, const char* gu_q, const char* gu_sm, const char* d_q,
                  const char* d_sm, size_t gu_q_b, size_t gu_sm_b, size_t d_q_b, size_t d_sm_b) {
  __shared__ Smem sm;
  DRB_TRACE_POINT(0, 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * ROWS_PER_BLOCK;
  const int nrows = min(ROWS_PER_BLOCK, E + 1 - row0);
  if (threadIdx.x == 0) {
    mbar_init(&sm.full, 1);
    mbar_fence_init();
    mbar_expect_tx(&sm.full, (unsigned)(nrows * K * 2));
    bulk_g2s(sm.w, W + (size_t)row0 * K, (unsigned)(nrows * K * 2), &sm.full);
  }
  __syncthreads();
  pdl_launch_dependents();  // the gate/up kernel may start fetching the shared expert's rows right away
  pdl_wait();               // x is the previous kernel's output
  DRB_TRACE_POINT(1, 0);

  // RMSNorm scale, recomputed by every block (8 KB of x from L2).
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4 xa = x4[threadIdx.x * 2], xb = x4[threadIdx.x * 2 + 1];  // k = 8*t .. 8*t+7
  float inv = 1.f;
  if (nw) {
    float ss = xa.x * xa.x + xa.y * xa.y + xa.z * xa.z + xa.w * xa.w + xb.x * xb.x + xb.y * xb.y + xb.z * xb.z + xb.w * xb.w;
    ss = warp_sum(ss);
    if (lane == 0) sm.red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += sm.red[w];
      sm.inv_rms = rsqrtf(t / K + eps);
    }
    __syncthreads();
    inv = sm.inv_rms;
  }
  unsigned long long xp[4];
  {
    float4 a = xa, b = xb;
    if (nw) {
      const float4 wa = reinterpret_cast<const float4*>(nw)[threadIdx.x * 2], wb = reinterpret_cast<const float4*>(nw)[threadIdx.x * 2 + 1];
      a = make_float4(a.x * inv * wa.x, a.y * inv * wa.y, a.z * inv * wa.z, a.w * inv * wa.w);
      b = make_float4(b.x * inv * wb.x, b.y * inv * wb.y, b.z * inv * wb.z, b.w * inv * wb.w);
    }
    xp[0] = pack2(a.x, a.y), xp[1] = pack2(a.z, a.w), xp[2] = pack2(b.x, b.y), xp[3] = pack2(b.z, b.w);
  }
  DRB_TRACE_POINT(2, 0);
  mbar_wait(&sm.full, 0, DRB_ERR_FULL_WAIT);
  DRB_TRACE_POINT(3, 0);
  // Each thread owns one 16-byte chunk (8 weights) of every row of the block.
#pragma unroll
  for (int r = 0; r < ROWS_PER_BLOCK; ++r) {
    float d = 0.f;
    if (r < nrows) {
      const uint4 v = *reinterpret_cast<const uint4*>(sm.w + (size_t)r * K * 2 + threadIdx.x * 16);
      float p0, p1;
      unpack2(dot8_bf16(v, xp, 0ull), p0, p1);
      d = p0 + p1;
    }
    d = warp_sum(d);
    if (lane == 0) sm.part[r][warp] = d;
  }
  __syncthreads();
  if ((int)threadIdx.x < nrows) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sm.part[threadIdx.x][w];
    __stcg(logits + row0 + threadIdx.x, t);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) sm.last = atomicAdd(counter, 1u) == gridDim.x - 1;
  __syncthreads();
  DRB_TRACE_POINT(4, 0);
  if (!sm.last) return;
  __threadfence();
  DRB_TRACE_ANY(5, 0);
  const int e = threadIdx.x;
  const float v = e < E ? __ldcg(logits + e) : -INFINITY;
  softmax_topk(v, E, topk, idx, wts, sm.tk);
  if (threadIdx.x == 0) {
    sgate[0] = __ldcg(logits + E);
    *counter = 0u;
  }
  DRB_TRACE_ANY(6, 0);
  // Optional: pull exactly the chosen experts into L2 (one bulk prefetch per region and expert).
  if (gu_q && threadIdx.x < 32) {
    __syncwarp();
    for (int i = threadIdx.x; i < topk * 4; i += 32) {
      const int k = i >> 2, which = i & 3;
      const size_t ex = (size_t)idx[k];
      const char* base = which == 0 ? gu_q : which == 1 ? gu_sm : which == 2 ? d_q : d_sm;
      const size_t nb = which == 0 ? gu_q_b : which == 1 ? gu_sm_b : which == 2 ? d_q_b : d_sm_b;
      if (base) prefetch_share(base + ex * nb, nb, 0, 1);
    }
  }
}

static cudaError_t configure_all() {
  cudaError_t e = drb_carveout(k_router_topk);
  if (e != cudaSuccess) return e;
  return drb_carveout(k_moe_topk);
}

}  // namespace router

// Reference: kernels/drama.cu:453-461; src/ffi.rs:56-60. K must be 2048, E <= 256, topk <= 32.
extern "C" int dr_router_topk(const __nv_bfloat16* W, const float* x, const float* nw, float eps, float* logits, int E,
                              int topk, int K, int* idx, float* wts, float* sgate, unsigned* counter, const char* gu_q,
                              const char* gu_sm, const char* d_q, const char* d_sm, size_t gu_q_b, size_t gu_sm_b,
                              size_t d_q_b, size_t d_sm_b, cudaStream_t st) {
  if (K != 2048 || E > 256 || E < 1 || topk > 32 || topk < 1 || topk > E) return -1;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  const int grid = (E + 1 + router::ROWS_PER_BLOCK - 1) / router::ROWS_PER_BLOCK;
  drb_launch(router::k_router_topk, dim3(grid), dim3(router::THREADS), 0, st, dev.pdl, W, x, nw, eps, logits, E, topk, idx,
             wts, sgate, counter, gu_q, gu_sm, d_q, d_sm, gu_q_b, gu_sm_b, d_q_b, d_sm_b);
  return 0;
}

// Reference: kernels/drama.cu:463-468; src/ffi.rs:41.
extern "C" int dr_moe_topk(const float* logits, int rows, int E, int topk, int stride, int* idx, float* wts, float* sgate,
                           cudaStream_t st) {
  if (E > 256 || E < 1 || topk > 32 || topk < 1 || topk > E) return -1;
  if (rows <= 0) return 0;
  const DrbDevice& dev = drb_device(st);
  if (!dev.ready) return -2;
  drb_launch(router::k_moe_topk, dim3(rows), dim3(router::THREADS), 0, st, dev.pdl, logits, E, topk, stride, idx, wts, sgate);
  return 0;
}
