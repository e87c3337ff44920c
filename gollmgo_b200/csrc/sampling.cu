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
// Logits crowd into a few values of the leading byte, so one shared histogram with atomics
// serialises (a millisecond per row at a vocabulary of 128 k).  Every warp keeps a histogram
// of its own instead: the lanes that fall into the same bin are found by comparison with a
// leader's bin, their weights are summed by the warp, and the leader adds the sum without an
// atomic; the warps' histograms are then added in warp order.  The sums therefore have a
// fixed order and the result is the same on every run.
template <bool MASS>
__device__ unsigned int radix_threshold(const float* row, int V, float m, float invT,
                                        unsigned int floor_key, float target, float* hist,
                                        float (*whist)[256]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  unsigned int prefix = 0, pmask = 0;
  float above = 0.f;       // weight of keys strictly above the current prefix range
  // In the first pass every element takes part and the bins of small values hold nearly all of
  // them, though the threshold is almost always within the three bins at and below the
  // maximum's.  So the first pass only bins those (`low_bin` = the lowest bin looked at); if
  // their weight does not reach the target, the pass is repeated over all bins.
  int low_bin = max(0, (int)(ordered_key(m) >> 24) - 2);
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (shift != 24) low_bin = 0;
    for (int i = lane; i < 256; i += 32) whist[warp][i] = 0.f;
    __syncwarp();
    // one element of every lane: the lanes of a bin are found by comparison with a leader's
    auto consume = [&](float x, bool valid) {
      int bin = -1;
      float w = 0.f;
      if (valid) {
        const unsigned int k = ordered_key(x);
        if (k >= floor_key && (k & pmask) == prefix && (int)((k >> shift) & 255u) >= low_bin) {
          bin = (int)((k >> shift) & 255u);
          w = MASS ? expf((x - m) * invT) : 1.f;
        }
      }
      unsigned todo = __ballot_sync(0xffffffffu, bin >= 0);
      while (todo) {
        const int leader = __ffs(todo) - 1;
        const int b = __shfl_sync(0xffffffffu, bin, leader);
        const bool mine = bin == b;
        const float sum = warp_sum(mine ? w : 0.f);
        if (lane == leader) whist[warp][b] += sum;
        todo &= ~__ballot_sync(0xffffffffu, mine);
      }
    };
    // four values per load where the row allows it: a quarter as many trips to L2 in a loop
    // whose votes keep the loads from overlapping
    const int V4 = (((size_t)row) & 15) == 0 ? V >> 2 : 0;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i0 = 0; i0 < V4; i0 += 4 * blockDim.x) {
      float4 v[4];
      bool valid[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {            // four loads in flight before the first vote
        const int i = i0 + u * blockDim.x + threadIdx.x;
        valid[u] = i < V4;
        v[u] = valid[u] ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        consume(v[u].x, valid[u]);
        consume(v[u].y, valid[u]);
        consume(v[u].z, valid[u]);
        consume(v[u].w, valid[u]);
      }
    }
    for (int i0 = V4 << 2; i0 < V; i0 += blockDim.x) {
      const int i = i0 + threadIdx.x;
      consume(i < V ? row[i] : 0.f, i < V);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      float v = 0.f;
      for (int wv = 0; wv < nw; ++wv) v += whist[wv][i];
      hist[i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float cum = above;
      int bin = 255;
      for (; bin > low_bin; --bin) {
        if (cum + hist[bin] >= target) break;
        cum += hist[bin];
      }
      // stopped at the lowest bin looked at without reaching the target: the bins below count too
      const bool again = low_bin > 0 && bin == low_bin && cum + hist[bin] < target;
      hist[256] = cum;
      hist[257] = __int_as_float(again ? -1 : bin);
    }
    __syncthreads();
    if (__float_as_int(hist[257]) < 0) {       // the same pass again over all bins
      __syncthreads();
      low_bin = 0;
      shift += 8;
      continue;
    }
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
  __shared__ float whist[SAMPLE_THREADS / 32][256];       // a histogram per warp (radix_threshold)
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
  if (k > 0 && k < V) floor_key = radix_threshold<false>(row, V, m, invT, 0u, (float)k, hist, whist);
  const float p = top_p ? top_p[r] : 0.f;
  if (p > 0.f && p < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = row[i];
      if (ordered_key(x) >= floor_key) z += expf((x - m) * invT);
    }
    z = block_sum(z, red_f);
    floor_key = radix_threshold<true>(row, V, m, invT, floor_key, p * z, hist, whist);
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
  gg_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, temperature, top_k, top_p, seeds, draw_index, out);
  return gg_check_launch("sample");
}
