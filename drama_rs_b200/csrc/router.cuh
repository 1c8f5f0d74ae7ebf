// Router: fused RMSNorm + bf16 router GEMV + softmax + top-k (dr_router_topk), and the
// prefill variant over precomputed logits (dr_moe_topk).
//
// Selection rule (the reference's, kernels/drama.cu:330-366 and 397-435): softmax over the E router
// logits in fp32, the k largest probabilities in descending order, ties to the lower expert index,
// weights divided by their sum accumulated in rank order; logit E is the shared-expert gate.
//
// The top-k is done without k serial arg-max rounds: the per-warp maxima give a lower bound for the
// selection, the few entries above it are ranked against each other through shared memory, and the ones
// whose rank is below k write themselves to their slot. Two block barriers instead of two per selected expert.
#pragma once

#include "common.cuh"

namespace router {

constexpr int THREADS = 256;  // one probability per thread in the tail: E <= 256
constexpr int MAX_TOPK = 32;

// a ranks before b: larger probability, or equal probability and lower index.
DRB_DEV bool before(float pa, int ia, float pb, int ib) { return pa > pb || (pa == pb && ia < ib); }

struct TopkSmem {
  float red[8];
  unsigned ured[8];
  int cnt[8];
  unsigned ukey[MAX_TOPK];
  __align__(16) unsigned long long comp[8 * MAX_TOPK];
  float top[MAX_TOPK];
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
// Built for latency: no serial arg-max rounds and no sort. Probabilities are >= 0, so their bit patterns order
// like unsigned integers; key = bits + 1 for a valid entry, 0 otherwise.
//   1. The largest logit of every warp is known from the softmax's max step. When at least topk warps hold valid
//      entries, the smallest of those maxima bounds the selection from below: topk entries are at least that large,
//      so nothing smaller can be selected. The bound is carried over to probabilities by pushing it through the
//      same exp and division every entry goes through (so entries that tie with it after rounding stay in).
//   2. The entries at or above the bound (typically two or three dozen of 256) go to shared memory as 64-bit
//      composites (key << 32 | ~index), whose plain unsigned order is "larger probability, then lower index";
//      their position comes from a ballot, not from a ranking.
//   3. Warp 0 ranks them against each other with shuffles (one survivor per lane; a loop over shared memory when
//      ties at the bound leave more than 32) and the ones whose rank is below topk write themselves to their slot.
// idx and wts are written by warp 0 only: other warps see them after the caller's next barrier.
// The softmax sums use the reference's reduction tree (kernels/drama.cu:39-47) so z has the same bits.
template <int BAR_ID = 0>
DRB_DEV void topk_sync() {
  if (BAR_ID == 0) __syncthreads();
  else asm volatile("bar.sync %0, 256;" ::"n"(BAR_ID) : "memory");
}

DRB_DEV float ord_to_float(unsigned o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o); }

// BAR_ID = 0: the block has exactly 256 threads. Otherwise threads 0..255 of a larger block call it and
// synchronise on named barrier BAR_ID.
// TK > 0 fixes topk at compile time; TK = 0 takes it from the argument.
template <int BAR_ID = 0, int TK = 0>
DRB_DEV void softmax_topk_impl(float v, int E, int topk, int* __restrict__ idx, float* __restrict__ wts, TopkSmem& sm) {
  if (TK > 0) topk = TK;
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  // max: one redux per warp on order-preserving integer keys, then eight values per thread
  const unsigned vb = __float_as_uint(v);
  const unsigned ord = (vb & 0x80000000u) ? ~vb : (vb | 0x80000000u);
  const unsigned wmax = __reduce_max_sync(0xffffffffu, ord);
  if (lane == 0) sm.ured[warp] = wmax;
  topk_sync<BAR_ID>();
  const int nvalid = (E + 31) >> 5;  // warps that hold valid entries
  unsigned mo = sm.ured[0], lo = sm.ured[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) {
    const unsigned u = sm.ured[w];
    mo = max(mo, u);
    if (w < nvalid) lo = min(lo, u);
  }
  const float m = ord_to_float(mo);
  const float ex = e < E ? expf(v - m) : 0.f;
  const float ws = warp_sum(ex);
  if (lane == 0) sm.red[warp] = ws;
  topk_sync<BAR_ID>();
  // the butterfly over the eight warp totals, written out: ((0+4)+(2+6)) + ((1+5)+(3+7))
  const float z = ((sm.red[0] + sm.red[4]) + (sm.red[2] + sm.red[6])) + ((sm.red[1] + sm.red[5]) + (sm.red[3] + sm.red[7]));
  const float p = e < E ? ex / z : -1.f;
  const unsigned key = e < E ? __float_as_uint(p) + 1u : 0u;
  unsigned bound = 1u;  // every valid entry
  if (nvalid >= topk) bound = __float_as_uint(expf(ord_to_float(lo) - m) / z) + 1u;
  // a warp's largest entry is always kept, so at least min(topk, valid warps) entries are, whatever exp rounds to
  const bool cand = key != 0u && (key >= bound || ord == wmax);
  const unsigned bal = __ballot_sync(0xffffffffu, cand);
  const unsigned long long mine = ((unsigned long long)key << 32) | (unsigned)(~e);
  if (cand) sm.comp[warp * MAX_TOPK + __popc(bal & ((1u << lane) - 1u))] = mine;
  if (lane == 0) sm.cnt[warp] = __popc(bal);
  topk_sync<BAR_ID>();
  // Warp 0 finishes alone. The survivors sit in (warp, lane) order, which is index order, so among equal keys
  // the earlier list position wins and 32-bit keys are all that has to travel.
  if (warp != 0) return;
  int off[9];
  off[0] = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) off[w + 1] = off[w] + sm.cnt[w];
  const int n = off[8];
  // survivor i sits in warp w's segment at position i - off[w]
  auto fetch = [&](int i) {
    int w = 0, ow = 0;
#pragma unroll
    for (int q = 1; q < 8; ++q) {
      const bool past = i >= off[q];
      w += past ? 1 : 0;
      ow = past ? off[q] : ow;
    }
    return sm.comp[w * MAX_TOPK + (i - ow)];
  };
  if (n <= 32) {
    // lane i takes survivor i; its rank is the number of survivors that come before it
    const unsigned long long c = lane < n ? fetch(lane) : 0ull;
    const unsigned k = (unsigned)(c >> 32);
    int r = 0;
#pragma unroll
    for (int o = 1; o < 32; ++o) {
      const int src = (lane + o) & 31;
      const unsigned ko = __shfl_sync(0xffffffffu, k, src);
      r += (ko > k || (ko == k && src < lane)) ? 1 : 0;
    }
    if (lane < n && r < topk) {
      idx[r] = (int)(~(unsigned)c);
      sm.top[r] = __uint_as_float(k - 1u);
    }
  } else {
    // many ties at the bound: every lane ranks its survivors against the whole list
    for (int i = lane; i < n; i += 32) {
      const unsigned long long c = fetch(i);
      int g = 0;
#pragma unroll
      for (int w2 = 0; w2 < 8; ++w2) {
        const int c2 = off[w2 + 1] - off[w2];
        for (int j = 0; j < c2; ++j) g += sm.comp[w2 * MAX_TOPK + j] > c ? 1 : 0;
      }
      if (g < topk) {
        idx[g] = (int)(~(unsigned)c);
        sm.top[g] = __uint_as_float((unsigned)(c >> 32) - 1u);
      }
    }
  }
  __syncwarp();
  if (lane < topk) {
    float total = 0.f;
    if (TK > 0) {
      float t[TK > 0 ? TK : 1];
#pragma unroll
      for (int k2 = 0; k2 < TK; ++k2) t[k2] = sm.top[k2];
#pragma unroll
      for (int k2 = 0; k2 < TK; ++k2) total += t[k2];  // rank order, as the reference accumulates
    } else {
      for (int k2 = 0; k2 < topk; ++k2) total += sm.top[k2];
    }
    wts[lane] = sm.top[lane] / total;
  }
  __syncwarp();
}

template <int BAR_ID = 0>
DRB_DEV void softmax_topk(float v, int E, int topk, int* __restrict__ idx, float* __restrict__ wts, TopkSmem& sm) {
  if (topk == 8) softmax_topk_impl<BAR_ID, 8>(v, E, topk, idx, wts, sm);
  else softmax_topk_impl<BAR_ID, 0>(v, E, topk, idx, wts, sm);
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
  const float v = (int)threadIdx.x < E ? __ldcg(l + threadIdx.x) : -INFINITY;
  softmax_topk(v, E, topk, idx + (size_t)r * topk, wts + (size_t)r * topk, sm);
  if (threadIdx.x == 0) sgate[r] = __ldcg(l + E);
}

constexpr int K = 2048;

// ------------------------------------------------------------------------------------------
// Decode router: ONE thread-block cluster of 8 blocks. Block c owns rows
// [33 c, 33 c + 33) of the [E+1, 2048] matrix and pulls them into shared memory with one bulk copy
// before the dependency wait; after the wait it normalises x, computes its logits and stores them
// straight into block 0's shared memory (distributed shared memory). One cluster barrier later block 0
// holds all E + 1 logits and runs the tail. No global atomics, no fences, no last-block election, and
// the counter word is never touched (so it stays zero, as the ABI requires).
namespace cl {

constexpr int CLUSTER = 8;
constexpr int ROWS = 33;                       // ceil(257 / 8)
constexpr int W_BYTES = ROWS * K * 2;          // 135,168
constexpr int CTL_BYTES = 4096;
constexpr size_t SMEM_BYTES = CTL_BYTES + K * 4 + W_BYTES;

struct Ctl {
  uint64_t full;
  float red[8];
  float inv_rms;
  float logits[CLUSTER * ROWS];  // block 0's copy is the gathering point
  TopkSmem tk;
};
static_assert(sizeof(Ctl) <= CTL_BYTES, "control block too large");

DRB_DEV unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `p` (a shared-memory address of this block) in block `rank`'s shared memory.
DRB_DEV uint32_t map_to_rank(const void* p, unsigned rank) {
  uint32_t d;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(smem_u32(p)), "r"(rank));
  return d;
}
DRB_DEV void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
DRB_DEV void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
DRB_DEV void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
    k_router_cluster(const __nv_bfloat16* __restrict__ W, const float* __restrict__ x, const float* __restrict__ nw, float eps,
                     float* __restrict__ logits, int E, int topk, int* __restrict__ idx, float* __restrict__ wts,
                     float* __restrict__ sgate, const char* gu_q, const char* gu_sm, const char* d_q, const char* d_sm,
                     size_t gu_q_b, size_t gu_sm_b, size_t d_q_b, size_t d_sm_b) {
  extern __shared__ __align__(128) unsigned char dyn[];
  Ctl& ctl = *reinterpret_cast<Ctl*>(dyn);
  float4* xs4 = reinterpret_cast<float4*>(dyn + CTL_BYTES);
  unsigned char* wsm = dyn + CTL_BYTES + K * 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned rank = cluster_rank();
  const int row0 = rank * ROWS;
  const int nrows = max(0, min(ROWS, E + 1 - row0));
  if (threadIdx.x == 0) {
    mbar_init(&ctl.full, 1);
    mbar_fence_init();
    if (nrows > 0) {
      mbar_expect_tx(&ctl.full, (unsigned)(nrows * K * 2));
      bulk_g2s(wsm, W + (size_t)row0 * K, (unsigned)(nrows * K * 2), &ctl.full);
    }
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();  // x is the previous kernel's output

  const float4 xa = __ldcg(reinterpret_cast<const float4*>(x) + threadIdx.x * 2), xb = __ldcg(reinterpret_cast<const float4*>(x) + threadIdx.x * 2 + 1);
  float inv = 1.f;
  float4 wa = make_float4(1.f, 1.f, 1.f, 1.f), wb = wa;
  if (nw) {
    wa = reinterpret_cast<const float4*>(nw)[threadIdx.x * 2], wb = reinterpret_cast<const float4*>(nw)[threadIdx.x * 2 + 1];
    float ss = xa.x * xa.x + xa.y * xa.y + xa.z * xa.z + xa.w * xa.w + xb.x * xb.x + xb.y * xb.y + xb.z * xb.z + xb.w * xb.w;
    ss = warp_sum(ss);
    if (lane == 0) ctl.red[warp] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += ctl.red[w];
    inv = rsqrtf(t / K + eps);
  }
  xs4[threadIdx.x * 2] = make_float4(xa.x * inv * wa.x, xa.y * inv * wa.y, xa.z * inv * wa.z, xa.w * inv * wa.w);
  xs4[threadIdx.x * 2 + 1] = make_float4(xb.x * inv * wb.x, xb.y * inv * wb.y, xb.z * inv * wb.z, xb.w * inv * wb.w);
  __syncthreads();
  // Warp w takes rows w, w + 8, ...; lane l takes the 16-byte chunks l, l + 32, ... (8 weights each) of a row.
  unsigned long long xp[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 a = xs4[2 * (lane + 32 * i)], b = xs4[2 * (lane + 32 * i) + 1];
    xp[4 * i] = pack2(a.x, a.y), xp[4 * i + 1] = pack2(a.z, a.w), xp[4 * i + 2] = pack2(b.x, b.y), xp[4 * i + 3] = pack2(b.z, b.w);
  }
  if (nrows > 0) mbar_wait(&ctl.full, 0, DRB_ERR_FULL_WAIT);
  const uint32_t gather = map_to_rank(ctl.logits, 0);
  // Four rows at a time per warp (rows warp, warp + 8, ...): independent accumulators, one folded reduction.
  for (int rb = warp; rb < nrows; rb += 32) {
    float d[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = rb + 8 * j;
      d[j] = 0.f;
      if (r < nrows) {
        const uint4* wr = reinterpret_cast<const uint4*>(wsm + (size_t)r * K * 2);
        unsigned long long a0 = 0ull, a1 = 0ull;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          a0 = dot8_bf16(wr[lane + 32 * i], xp + 4 * i, a0);
          a1 = dot8_bf16(wr[lane + 32 * (i + 1)], xp + 4 * (i + 1), a1);
        }
        float p0, p1, p2, p3;
        unpack2(a0, p0, p1);
        unpack2(a1, p2, p3);
        d[j] = (p0 + p1) + (p2 + p3);
      }
    }
    const bool hi16 = lane & 16, hi8 = lane & 8;
    const float r0 = (hi16 ? d[2] : d[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? d[0] : d[2], 16);
    const float r1 = (hi16 ? d[3] : d[1]) + __shfl_xor_sync(0xffffffffu, hi16 ? d[1] : d[3], 16);
    float sres = (hi8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi8 ? r0 : r1, 8);
    sres += __shfl_xor_sync(0xffffffffu, sres, 4);
    sres += __shfl_xor_sync(0xffffffffu, sres, 2);
    sres += __shfl_xor_sync(0xffffffffu, sres, 1);
    const int r = rb + 8 * (lane >> 3);  // lanes 0-7: row j = 0, 8-15: j = 1, 16-23: j = 2, 24-31: j = 3
    if ((lane & 7) == 0 && r < nrows) st_cluster_f32(gather + 4u * (unsigned)(row0 + r), sres);
  }
  cluster_arrive();
  if (rank != 0) return;  // only block 0's shared memory is read from here on
  cluster_wait();
  const int e = threadIdx.x;
  const float v = e < E ? ctl.logits[e] : -INFINITY;
  if (e < E) logits[e] = v;
  if (e == 0) logits[E] = ctl.logits[E];
  softmax_topk(v, E, topk, idx, wts, ctl.tk);
  if (threadIdx.x == 0) sgate[0] = ctl.logits[E];
  if (gu_q && threadIdx.x < 32) {
    __syncwarp();
    // Pull exactly the chosen experts into L2: region `which` of expert idx[k], cut into bulk prefetches.
    for (int i = threadIdx.x; i < topk * 4; i += 32) {
      const int k = i >> 2, which = i & 3;
      const size_t ex = (size_t)idx[k];
      const char* base = which == 0 ? gu_q : which == 1 ? gu_sm : which == 2 ? d_q : d_sm;
      const size_t nb = which == 0 ? gu_q_b : which == 1 ? gu_sm_b : which == 2 ? d_q_b : d_sm_b;
      if (base) prefetch_share(base + ex * nb, nb, 0, 1);
    }
  }
}

}  // namespace cl

static cudaError_t configure_all() {
  cudaError_t e = drb_carveout(cl::k_router_cluster);
  if (e != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(cl::k_router_cluster, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cl::SMEM_BYTES)) != cudaSuccess) return e;
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
  // One cluster of 8 blocks, launched with the programmatic-dependency attribute as well. The counter word of the
  // ABI is never touched (it stays zero, as the caller expects): nothing here needs a last-block election.
  (void)counter;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(router::cl::CLUSTER);
  cfg.blockDim = dim3(router::THREADS);
  cfg.dynamicSmemBytes = router::cl::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = router::cl::CLUSTER, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dev.pdl ? 2 : 1;
  cudaLaunchKernelEx(&cfg, router::cl::k_router_cluster, W, x, nw, eps, logits, E, topk, idx, wts, sgate, gu_q, gu_sm, d_q,
                     d_sm, gu_q_b, gu_sm_b, d_q_b, d_sm_b);
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
