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

// The common case at full width: bfloat16, half-split pairs, the whole head rotated, head size a
// multiple of 16.  One CTA per token; a thread takes eight pairs of one head with two 16-byte
// loads (columns p..p+7 and p+d/2..p+d/2+7), or eight values of a v head, and stores in kind.
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                         const int* __restrict__ slot_mapping, const double* __restrict__ inv_freq,
                         __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int nh, int nkv,
                         int d, int page_size, int write_cache) {
  extern __shared__ float cs[];        // cos[d/2], sin[d/2]
  pdl_trigger();
  const int t = blockIdx.x;
  const int half = d >> 1;
  // The token's position and cache slot were copied in before the step began and the
  // frequencies never change: the table of cosines and sines is ready before the kernel
  // ahead (the qkv product) has finished; only the rows of qkv have to wait for it.
  {
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
  const int slot = (write_cache && slot_mapping) ? slot_mapping[t] : -1;
  __syncthreads();
  pdl_wait();
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  __nv_bfloat16* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
  const int per_head = half >> 3;                       // groups of eight pairs per head
  const int rot_items = (nh + nkv) * per_head, v_items = nkv * (d >> 3);
  for (int e = threadIdx.x; e < rot_items + v_items; e += blockDim.x) {
    if (e < rot_items) {
      const int h = e / per_head, p0 = (e - h * per_head) << 3;
      __nv_bfloat16* x = row + (size_t)h * d;
      uint4 lo = *reinterpret_cast<const uint4*>(x + p0), hi = *reinterpret_cast<const uint4*>(x + half + p0);
      __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&lo);
      __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(a2[i]), b = __bfloat1622float2(b2[i]);
        const float c0 = cs[p0 + 2 * i], s0 = cs[half + p0 + 2 * i], c1 = cs[p0 + 2 * i + 1], s1 = cs[half + p0 + 2 * i + 1];
        a2[i] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
        b2[i] = __floats2bfloat162_rn(a.x * s0 + b.x * c0, a.y * s1 + b.y * c1);
      }
      *reinterpret_cast<uint4*>(x + p0) = lo;
      *reinterpret_cast<uint4*>(x + half + p0) = hi;
      if (h >= nh && slot >= 0) {
        __nv_bfloat16* kc = kcache + (((size_t)page * nkv + (h - nh)) * page_size + off) * d;
        *reinterpret_cast<uint4*>(kc + p0) = lo;
        *reinterpret_cast<uint4*>(kc + half + p0) = hi;
      }
    } else if (slot >= 0) {
      const int ev = e - rot_items;
      const int h = ev / (d >> 3), c = (ev - h * (d >> 3)) << 3;
      *reinterpret_cast<uint4*>(vcache + (((size_t)page * nkv + h) * page_size + off) * d + c) =
          *reinterpret_cast<const uint4*>(row + (size_t)(nh + nkv + h) * d + c);
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
  if (act_dtype == GG_BF16 && inv_freq && rot == d && d % 16 == 0 && !interleaved &&
      ((size_t)qkv % 16) == 0 && (!write_cache || (((size_t)kcache % 16) == 0 && ((size_t)vcache % 16) == 0))) {
    gg_launch(rope_kv_write_vec_kernel, dim3(T), dim3(256), smem, stream, (__nv_bfloat16*)qkv, positions, slot_mapping,
              inv_freq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, nkv, d, page_size, write_cache);
    return gg_check_launch("rope_kv_write");
  }
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
