// Token selection from float32 logits, one thread block per row.
//
// Follows internal/engine/sampling.go:40-192 of the reference (which samples on
// the host in float64): temperature <= 1e-9 means greedy (first maximum wins);
// otherwise logits/T, keep the top_k largest (0 = off), softmax, keep the
// smallest sorted prefix whose mass reaches top_p (0 or >= 1 = off), renormalise,
// and take the first index whose running sum exceeds a uniform draw.  The draw
// of request r for its n-th token is a counter-based hash of (seed_r, n), so a
// request's tokens do not depend on what else is in the batch.
// Elements equal to the top-k or top-p threshold value are all kept.
#include "common.cuh"
#include <cstring>
#include <cstdlib>

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned int ordered_key(float x) {
  unsigned int b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float uniform_draw(unsigned long long seed, unsigned long long n) {
  unsigned long long z = seed + (n + 1ULL) * 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// First index of the maximum of row[0..V).
__device__ int block_argmax(const float* row, int V, float* red_f, int* red_i, float* max_out) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if ((((size_t)row) & 15) == 0) {
    // four values per load; within a thread indices only grow, so ">" keeps the first maximum
    const int V4 = V >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
      const float4 v = row4[i];
      if (v.x > best) { best = v.x; bi = 4 * i; }
      if (v.y > best) { best = v.y; bi = 4 * i + 1; }
      if (v.z > best) { best = v.z; bi = 4 * i + 2; }
      if (v.w > best) { best = v.w; bi = 4 * i + 3; }
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  __syncthreads();
  if (lane == 0) { red_f[warp] = best; red_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? red_f[lane] : -INFINITY;
    bi = lane < nw ? red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { red_f[32] = best; red_i[32] = bi; }
  }
  __syncthreads();
  if (max_out) *max_out = red_f[32];
  return red_i[32] == 0x7fffffff ? 0 : red_i[32];
}

__global__ void argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
  __shared__ float red_f[33];
  __shared__ int red_i[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int idx = block_argmax(logits + (size_t)r * V, V, red_f, red_i, nullptr);
  if (threadIdx.x == 0) out[r] = idx;
}

// Radix descent from the most significant byte: the key K such that the elements
// with key > K weigh less than `target` and those with key >= K weigh at least
// `target`.  weight(i) = 1 (count mode, the k-th largest) or exp((x_i - m) * invT)
// (mass mode).  Only elements with key >= floor_key take part.
// Leading byte: logits crowd into a few of its values (one shared histogram with atomics
// serialised there: a millisecond per row at a vocabulary of 128 k), and the threshold is
// almost always within the three values at and below the maximum's.  So a thread first adds up
// the weights of its elements in just those three bins, in registers, and the block adds the
// threads' sums in a fixed order.  Only if the three bins together do not reach the target is
// the leading byte binned in full.  Lower bytes (and that full pass): the elements still in the
// range spread over many bins; atomic adds on a histogram of 64-bit integers (weights in fixed
// point, 40 fraction bits).  Integer sums do not depend on their order and the others have a
// fixed one, so the result is the same on every run.
// ---- a row spread over the CTAs of a thread-block cluster (sample_cluster_kernel): what a
// CTA shows its neighbours.  Two copies, used in turn: a copy is written again only after a
// further cluster barrier, which nobody passes before everybody has read the one before.
struct ClusterPub {
  float hist[2][256];
  float f[2];
  int i[2];
  int parity;            // which copy the next exchange uses (the same in every CTA)
};
__device__ __forceinline__ unsigned sc_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned sc_size() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sc_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T> __device__ __forceinline__ T sc_load(const T* local, unsigned rank) {
  unsigned v, a = (unsigned)__cvta_generic_to_shared(local);
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %1, %2;\n\t"
      "ld.shared::cluster.b32 %0, [ra];\n\t}"
      : "=r"(v) : "r"(a), "r"(rank) : "memory");
  T out;
  memcpy(&out, &v, 4);
  return out;
}

// CL: row is this CTA's part of the row and the histogram of a pass is the sum over the
// cluster's CTAs in rank order, the same in every CTA, so every CTA descends alike.
template <bool MASS, bool CL>
__device__ unsigned int radix_threshold(const float* row, int V, float m, float invT,
                                        unsigned int floor_key, float target, float* hist,
                                        float* red, unsigned long long* h64, ClusterPub* pub = nullptr) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float FX = 1099511627776.f;        // 2^40
  unsigned int prefix = 0, pmask = 0;
  float above = 0.f;       // weight of keys strictly above the current prefix range
  // every element of the row (or of this CTA's part of it), four per load where possible
  auto for_each = [&](auto&& f) {
    const int V4 = (((size_t)row) & 15) == 0 ? V >> 2 : 0;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
      const float4 v = row4[i];
      f(v.x); f(v.y); f(v.z); f(v.w);
    }
    for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) f(row[i]);
  };
  // hist[0..n) = the block's (CL: the cluster's) sum of hist[0..n) as every thread sees it
  auto exchange = [&](int n) {
    if (CL) {
      const int par = pub->parity;
      for (int i = threadIdx.x; i < n; i += blockDim.x) pub->hist[par][i] = hist[i];
      sc_barrier();                            // (also a barrier of the CTA)
      const unsigned C = sc_size();
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = 0.f;
        for (unsigned c = 0; c < C; ++c) v += sc_load(&pub->hist[par][i], c);
        hist[i] = v;
      }
      __syncthreads();
      if (threadIdx.x == 0) pub->parity = par ^ 1;
    }
    __syncthreads();
  };
  // ---- leading byte, the three bins at and below the maximum's
  const int top = (int)(ordered_key(m) >> 24);
  bool full = true;                            // the leading byte still has to be binned in full
  {
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
    for_each([&](float x) {
      const unsigned int k = ordered_key(x);
      const int d = top - (int)(k >> 24);
      if (k >= floor_key && d >= 0 && d <= 2) {
        const float w = MASS ? expf((x - m) * invT) : 1.f;
        if (d == 0) acc0 += w; else if (d == 1) acc1 += w; else acc2 += w;
      }
    });
    acc0 = block_sum(acc0, red);
    acc1 = block_sum(acc1, red);
    acc2 = block_sum(acc2, red);
    if (threadIdx.x == 0) { hist[0] = acc0; hist[1] = acc1; hist[2] = acc2; }
    __syncthreads();
    exchange(3);
    float cum = 0.f;
    for (int d = 0; d <= 2 && d <= top; ++d) {
      if (cum + hist[d] >= target) {
        prefix = (unsigned int)(top - d) << 24;
        pmask = 255u << 24;
        above = cum;
        full = false;
        break;
      }
      cum += hist[d];
    }
    __syncthreads();                           // hist is written again below
  }
  for (int shift = full ? 24 : 16; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) h64[i] = 0ULL;
    __syncthreads();
    for_each([&](float x) {
      const unsigned int k = ordered_key(x);
      if (k >= floor_key && (k & pmask) == prefix) {
        const unsigned long long w = MASS ? (unsigned long long)(expf((x - m) * invT) * FX) : 1ULL;
        atomicAdd(h64 + ((k >> shift) & 255u), w);
      }
    });
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += blockDim.x)
      hist[i] = MASS ? (float)h64[i] * (1.f / FX) : (float)h64[i];
    __syncthreads();
    exchange(256);
    if (warp == 0) {
      // the first bin from the top whose weight, added to that of the bins above, reaches the
      // target (bin 0 where none does).  Lane l takes bins 255 - 8 l down to 248 - 8 l: one
      // thread walking 256 bins is 256 dependent reads of shared memory, 4 us a pass.
      float hs[8], s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int b = 255 - 8 * lane - j;
        hs[j] = b > 0 ? hist[b] : 0.f;
        s += hs[j];
      }
      float incl = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      float cum = above + (incl - s);
      int fb = -1;
      float fcum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int b = 255 - 8 * lane - j;
        if (b > 0 && fb < 0) {
          if (cum + hs[j] >= target) { fb = b; fcum = cum; }
          else cum += hs[j];
        }
      }
      const unsigned any = __ballot_sync(0xffffffffu, fb >= 0);
      const int src = any ? __ffs(any) - 1 : 31;
      const int bin = any ? __shfl_sync(0xffffffffu, fb, src) : 0;
      const float all = __shfl_sync(0xffffffffu, incl, 31);
      const float cumv = any ? __shfl_sync(0xffffffffu, fcum, src) : above + all;
      if (lane == 0) {
        hist[256] = cumv;
        hist[257] = __int_as_float(bin);
      }
    }
    __syncthreads();
    above = hist[256];
    const unsigned int bin = (unsigned int)__float_as_int(hist[257]);
    prefix |= bin << shift;
    pmask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ draw_index, int* __restrict__ out) {
  __shared__ float red_f[33];
  __shared__ int red_i[33];
  __shared__ float hist[258];
  __shared__ unsigned long long h64[256];
  __shared__ float scan[SAMPLE_THREADS / 32 + 1];
  __shared__ int found;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float T = temperature[r];
  float m;
  const int amax = block_argmax(row, V, red_f, red_i, &m);
  if (T <= 1e-9f) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  const float invT = 1.f / T;
  unsigned int floor_key = 0;
  const int k = top_k ? top_k[r] : 0;
  if (k > 0 && k < V) floor_key = radix_threshold<false, false>(row, V, m, invT, 0u, (float)k, hist, red_f, h64);
  const float p = top_p ? top_p[r] : 0.f;
  if (p > 0.f && p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = row[i];
      if (ordered_key(x) >= floor_key) z += expf((x - m) * invT);
    }
    z = block_sum(z, red_f);
    floor_key = radix_threshold<true, false>(row, V, m, invT, floor_key, p * z, hist, red_f, h64);
  }
  // running sum in index order over the kept elements; thread owns a contiguous chunk
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int i0 = min(V, (int)threadIdx.x * chunk), i1 = min(V, i0 + chunk);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = row[i];
    if (ordered_key(x) >= floor_key) local += expf((x - m) * invT);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (threadIdx.x == 0) found = -1;
  if (lane == 31) scan[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; ++w) { const float v = scan[w]; scan[w] = run; run += v; }
    scan[nw] = run;
  }
  __syncthreads();
  const float total = scan[blockDim.x >> 5];
  const float before = scan[warp] + incl - local;
  const float u = uniform_draw(seeds ? seeds[r] : 0ULL, draw_index ? draw_index[r] : 0ULL);
  const float target = u * total;
  if (local > 0.f && target >= before && target < before + local) {
    float cum = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float x = row[i];
      if (ordered_key(x) >= floor_key) {
        cum += expf((x - m) * invT);
        pick = i;
        if (target < cum) break;
      }
    }
    if (pick >= 0) atomicMax(&found, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = found >= 0 ? found : amax;
}

// ---------------------------------------------------------------- a row on a cluster of CTAs
// One CTA per row reads its 128 k logits from L2 a dozen times (maximum, top-k and top-p
// descents of up to four passes each, sums), at the rate one SM gets from L2: 266 us with top-k
// and top-p before the descent was rewritten (43 us here, for 8 rows).  Here a row is cut into SC_CLUSTER parts, one per CTA of a cluster; a CTA reads
// its part from global memory once and keeps it in shared memory, and the CTAs exchange
// histograms and sums through distributed shared memory, always added in rank order, so every
// CTA takes the same decisions and the result is the same on every run.  Same arithmetic per
// element as sample_kernel; sums are associated differently (parts instead of 1024 strides).
#define SC_THREADS 512
#define SC_CLUSTER 8
#define SC_MIN_V 16384            // shorter rows stay with sample_kernel

// sum of v over the cluster in rank order (every CTA gets the same bits); *before = the sum
// over the ranks below this CTA's.  Called by all threads; v of thread 0 counts.
__device__ float sc_sum(float v, ClusterPub* pub, float* bcast, float* before) {
  const int par = pub->parity;
  if (threadIdx.x == 0) pub->f[par] = v;
  sc_barrier();
  if (threadIdx.x == 0) {
    const unsigned C = sc_size(), me = sc_rank();
    float run = 0.f, mine = 0.f;
    for (unsigned c = 0; c < C; ++c) {
      if (c == me) mine = run;
      run += sc_load(&pub->f[par], c);
    }
    bcast[0] = run;
    bcast[1] = mine;
    pub->parity = par ^ 1;
  }
  __syncthreads();
  if (before) *before = bcast[1];
  return bcast[0];
}

__global__ void __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int V, int part, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                      const unsigned long long* __restrict__ seeds,
                      const unsigned long long* __restrict__ draw_index, int* __restrict__ out) {
  extern __shared__ __align__(16) float sc_part[];          // this CTA's part of the row
  __shared__ float red_f[33];
  __shared__ int red_i[33];
  __shared__ float hist[258];
  __shared__ unsigned long long h64[256];
  __shared__ float scan[SC_THREADS / 32 + 1];
  __shared__ float bcast[2];
  __shared__ int found;
  __shared__ ClusterPub pub;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const unsigned me = sc_rank(), C = sc_size();
  const int base = (int)me * part, n = max(0, min(part, V - base));   // elements [base, base + n)
  const float* row = logits + (size_t)r * V;
  if (threadIdx.x == 0) pub.parity = 0;
  // the part into shared memory (float4 where the row's start allows it; part is a multiple of 4)
  if (((((size_t)row) & 15) == 0) && (n & 3) == 0) {
    const float4* src = reinterpret_cast<const float4*>(row + base);
    float4* dst = reinterpret_cast<float4*>(sc_part);
    for (int i = threadIdx.x; i < (n >> 2); i += SC_THREADS) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < n; i += SC_THREADS) sc_part[i] = row[base + i];
  }
  __syncthreads();
  const float T = temperature[r];
  // the maximum and its first index: of the part, then of the row (the lowest rank wins a tie)
  float m_local;
  const int a_local = block_argmax(sc_part, n, red_f, red_i, &m_local);
  if (threadIdx.x == 0) { pub.f[0] = n > 0 ? m_local : -INFINITY; pub.i[0] = base + a_local; }
  sc_barrier();
  float m = -INFINITY;
  int amax = 0;
  for (unsigned c = 0; c < C; ++c) {
    const float v = sc_load(&pub.f[0], c);
    if (v > m) { m = v; amax = sc_load(&pub.i[0], c); }
  }
  __syncthreads();
  if (threadIdx.x == 0) pub.parity = 1;
  __syncthreads();
  if (T <= 1e-9f) {
    if (me == 0 && threadIdx.x == 0) out[r] = amax;
    sc_barrier();                            // nobody leaves while a neighbour may still read it
    return;
  }
  const float invT = 1.f / T;
  unsigned int floor_key = 0;
  const int k = top_k ? top_k[r] : 0;
  if (k > 0 && k < V) floor_key = radix_threshold<false, true>(sc_part, n, m, invT, 0u, (float)k, hist, red_f, h64, &pub);
  const float p = top_p ? top_p[r] : 0.f;
  if (p > 0.f && p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < n; i += SC_THREADS) {
      const float x = sc_part[i];
      if (ordered_key(x) >= floor_key) z += expf((x - m) * invT);
    }
    z = block_sum(z, red_f);
    z = sc_sum(z, &pub, bcast, nullptr);
    floor_key = radix_threshold<true, true>(sc_part, n, m, invT, floor_key, p * z, hist, red_f, h64, &pub);
  }
  // running sum in index order over the kept elements: a thread owns a contiguous piece of
  // the part, a CTA the part, the ranks follow each other
  const int chunk = ((n + SC_THREADS - 1) / SC_THREADS) | 1;      // odd: the lanes' pieces start in different banks
  const int i0 = min(n, (int)threadIdx.x * chunk), i1 = min(n, i0 + chunk);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = sc_part[i];
    if (ordered_key(x) >= floor_key) local += expf((x - m) * invT);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (threadIdx.x == 0) found = -1;
  if (lane == 31) scan[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int w = 0; w < SC_THREADS / 32; ++w) { const float v = scan[w]; scan[w] = run; run += v; }
    scan[SC_THREADS / 32] = run;
  }
  __syncthreads();
  float ranks_before;
  const float total = sc_sum(scan[SC_THREADS / 32], &pub, bcast, &ranks_before);
  const float before = ranks_before + scan[warp] + incl - local;
  const float u = uniform_draw(seeds ? seeds[r] : 0ULL, draw_index ? draw_index[r] : 0ULL);
  const float target = u * total;
  if (local > 0.f && target >= before && target < before + local) {
    float cum = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float x = sc_part[i];
      if (ordered_key(x) >= floor_key) {
        cum += expf((x - m) * invT);
        pick = base + i;
        if (target < cum) break;
      }
    }
    if (pick >= 0) atomicMax(&found, pick);
  }
  __syncthreads();
  // the largest index anybody found (rounding can make two neighbours claim the draw, or
  // nobody: then the maximum's index, as in sample_kernel)
  const int par = pub.parity;
  if (threadIdx.x == 0) pub.i[par] = found;
  sc_barrier();
  if (me == 0 && threadIdx.x == 0) {
    int best = -1;
    for (unsigned c = 0; c < C; ++c) best = max(best, sc_load(&pub.i[par], c));
    out[r] = best >= 0 ? best : amax;
  }
  sc_barrier();                              // nobody leaves while rank 0 may still read it
}

extern "C" int gg_argmax(const float* logits, int R, int V, int* out, cudaStream_t stream) {
  GG_REQUIRE(R >= 0 && V > 0, "argmax: bad sizes R=%d V=%d", R, V);
  if (R == 0) return GG_OK;
  gg_launch(argmax_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, out);
  return gg_check_launch("argmax");
}

extern "C" int gg_sample(const float* logits, int R, int V, const float* temperature,
                         const int* top_k, const float* top_p, const unsigned long long* seeds,
                         const unsigned long long* draw_index, int* out, cudaStream_t stream) {
  GG_REQUIRE(R >= 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
  GG_REQUIRE(temperature != nullptr, "sample: no temperatures given");
  if (R == 0) return GG_OK;
  static int use_cluster = -1;
  if (use_cluster < 0) { const char* e = getenv("GOLLMGO_B200_SAMPLE_CLUSTER"); use_cluster = e ? atoi(e) : 1; }
  const int part = (((V + SC_CLUSTER - 1) / SC_CLUSTER) + 3) & ~3;
  const size_t smem = (size_t)part * sizeof(float);
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  // (with more rows than clusters fit at once, two CTAs per SM, a CTA per row is about as fast:
  // 64 rows with top-k and top-p 158 against 145 us, temperature only 43 against 59; 8 rows: 43 us
  // on clusters against 120 with a CTA per row)
  if (use_cluster && V >= SC_MIN_V && smem <= 160 * 1024 && R * SC_CLUSTER <= 2 * num_sms) {
    static bool set = false;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "sample: %s", cudaGetErrorString(e));
      set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SC_CLUSTER, R);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SC_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gg_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, V, part, temperature, top_k, top_p, seeds, draw_index, out);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "sample: launch: %s", cudaGetErrorString(e));
    return gg_check_launch("sample");
  }
  gg_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, temperature, top_k, top_p, seeds, draw_index, out);
  return gg_check_launch("sample");
}
