// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// Reference: kernels/gollmgo_ops.cu:321-358 (rope, adjacent pairs, theta fixed at
// 10000) followed by kernels/gollmgo_paged_attn.cu:126-146 (scatter by slot).  Here
// the inverse frequencies come from a table the host builds from config.json
// (theta, rope_scaling), the pairing is half-split (p, p+rot/2) unless
// `interleaved`, and one kernel does both so k and v are read once.
//
// qkv:   [T, (nh + 2*nkv) * d]   q heads, then k heads, then v heads; q and k are
//        rotated in place (k also lands rotated in the cache)
// cache: K and V of one layer, each [num_pages, nkv, page_size, d]
// slot:  slot_mapping[t] = page * page_size + offset, or < 0 to skip the write
// inv_freq: rot/2 doubles, or null for no rotation (then only the cache write happens)
// The angle pos * inv_freq is formed and reduced modulo 2 pi in float64; sine, cosine
// and the rotation itself are float32.
#include "common.cuh"

#define ROPE_HEADS_PER_CTA 8

// grid (T, ceil((nh + 2 nkv) / 8)): a CTA takes eight consecutive heads (q, k or v) of one token.
template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping,
                                     const double* __restrict__ inv_freq, TA* __restrict__ kcache,
                                     TA* __restrict__ vcache, int nh, int nkv, int d, int rot,
                                     int page_size, int interleaved, int write_cache) {
  extern __shared__ float cs[];        // cos[rot/2], sin[rot/2]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const int h0 = blockIdx.y * ROPE_HEADS_PER_CTA;
  const int h1 = min(h0 + ROPE_HEADS_PER_CTA, nh + 2 * nkv);
  const bool rotates = inv_freq && h0 < nh + nkv;
  if (rotates) {
    // angle in float64, reduced to [-pi, pi] in float64, then float32 sine and cosine: the
    // reduction keeps the accuracy of the float64 product at any position, and the float32
    // functions are exact to an ulp on the reduced argument
    const double pos = (double)positions[t];
    const double two_pi = 6.283185307179586476925286766559;
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
      const double ang = pos * inv_freq[p];
      const float r = (float)(ang - two_pi * rint(ang * (1.0 / two_pi)));
      float s, c;
      sincosf(r, &s, &c);
      cs[p] = c;
      cs[half + p] = s;
    }
  }
  __syncthreads();
  const int slot = (write_cache && slot_mapping) ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  TA* row = qkv + (size_t)t * (nh + 2 * nkv) * d;

  for (int h = h0; h < h1; ++h) {
    TA* x = row + (size_t)h * d;
    if (h < nh + nkv) {
      // a q or k head: rotate `half` pairs, copy the rest of a k head to the cache as it is
      TA* kc = (h >= nh && slot >= 0) ? kcache + (((size_t)page * nkv + (h - nh)) * page_size + off) * d : nullptr;
      if (inv_freq) {
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
          const int i0 = interleaved ? 2 * p : p;
          const int i1 = interleaved ? 2 * p + 1 : p + half;
          const float a = to_f32(x[i0]), b = to_f32(x[i1]);
          const float c = cs[p], s = cs[half + p];
          const TA ra = from_f32<TA>(a * c - b * s);
          const TA rb = from_f32<TA>(a * s + b * c);
          x[i0] = ra;
          x[i1] = rb;
          if (kc) { kc[i0] = ra; kc[i1] = rb; }
        }
      }
      if (kc) {
        const int from = inv_freq ? rot : 0;
        for (int c = from + threadIdx.x; c < d; c += blockDim.x) kc[c] = x[c];
      }
    } else if (slot >= 0) {
      TA* vcp = vcache + (((size_t)page * nkv + (h - nh - nkv)) * page_size + off) * d;
      for (int c = threadIdx.x; c < d; c += blockDim.x) vcp[c] = x[c];
    }
  }
}

extern "C" int gg_rope_kv_write(void* qkv, int act_dtype, const int* positions,
                                const int* slot_mapping, const double* inv_freq, void* kcache,
                                void* vcache, int T, int nh, int nkv, int d, int rot,
                                int page_size, int interleaved, int write_cache,
                                cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && d > 0 && page_size > 0,
             "rope_kv_write: bad sizes T=%d nh=%d nkv=%d d=%d page=%d", T, nh, nkv, d, page_size);
  GG_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_kv_write: rotary width %d must be even and <= head size %d", rot, d);
  GG_REQUIRE(!write_cache || (kcache && vcache && slot_mapping), "rope_kv_write: cache write without cache or slots");
  if (T == 0) return GG_OK;
  if (rot == 0) inv_freq = nullptr;
  const size_t smem = (size_t)rot * sizeof(float);
  GG_REQUIRE(smem <= 48 * 1024, "rope_kv_write: rotary width %d too large", rot);
  const int threads = d >= 256 ? 128 : 64;
  const dim3 grid(T, (nh + 2 * nkv + ROPE_HEADS_PER_CTA - 1) / ROPE_HEADS_PER_CTA);
  GG_REQUIRE(grid.y <= 65535, "rope_kv_write: too many heads");
  if (act_dtype == GG_F32)
    gg_launch(rope_kv_write_kernel<float>, grid, dim3(threads), smem, stream, (float*)qkv, positions, slot_mapping, inv_freq, (float*)kcache, (float*)vcache, nh, nkv, d, rot, page_size, interleaved, write_cache);
  else if (act_dtype == GG_BF16)
    gg_launch(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, (__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, nkv, d, rot, page_size, interleaved, write_cache);
  else
    return gg_fail(GG_ERR_INVALID, "rope_kv_write: unknown dtype %d", act_dtype);
  return gg_check_launch("rope_kv_write");
}
