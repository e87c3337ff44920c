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
// The angle pos * inv_freq and its sine/cosine are evaluated in float64, the
// rotation itself in float32.
#include "common.cuh"

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
  if (inv_freq) {
    const double pos = (double)positions[t];
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
      double s, c;
      sincos(pos * inv_freq[p], &s, &c);
      cs[p] = (float)c;
      cs[half + p] = (float)s;
    }
  }
  __syncthreads();
  const int slot = (write_cache && slot_mapping) ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  TA* row = qkv + (size_t)t * (nh + 2 * nkv) * d;

  if (inv_freq) {
    // q and k heads: (nh + nkv) * half rotation pairs
    const int npairs = (nh + nkv) * half;
    for (int e = threadIdx.x; e < npairs; e += blockDim.x) {
      const int h = e / half, p = e - h * half;
      TA* x = row + (size_t)h * d;
      const int i0 = interleaved ? 2 * p : p;
      const int i1 = interleaved ? 2 * p + 1 : p + half;
      const float a = to_f32(x[i0]), b = to_f32(x[i1]);
      const float c = cs[p], s = cs[half + p];
      const TA ra = from_f32<TA>(a * c - b * s);
      const TA rb = from_f32<TA>(a * s + b * c);
      x[i0] = ra;
      x[i1] = rb;
      if (h >= nh && slot >= 0) {
        TA* kc = kcache + (((size_t)page * nkv + (h - nh)) * page_size + off) * d;
        kc[i0] = ra;
        kc[i1] = rb;
      }
    }
  }
  if (slot >= 0) {
    // the part of k that is not rotated (all of it when there is no table), and v
    const int krest = inv_freq ? d - rot : d;
    const int kfrom = inv_freq ? rot : 0;
    for (int e = threadIdx.x; e < nkv * krest; e += blockDim.x) {
      const int h = e / krest, c = kfrom + (e - h * krest);
      kcache[(((size_t)page * nkv + h) * page_size + off) * d + c] = row[(size_t)(nh + h) * d + c];
    }
    for (int e = threadIdx.x; e < nkv * d; e += blockDim.x) {
      const int h = e / d, c = e - h * d;
      vcache[(((size_t)page * nkv + h) * page_size + off) * d + c] = row[(size_t)(nh + nkv + h) * d + c];
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
  const int threads = 256;
  if (act_dtype == GG_F32)
    gg_launch(rope_kv_write_kernel<float>, dim3(T), dim3(threads), smem, stream, (float*)qkv, positions, slot_mapping, inv_freq, (float*)kcache, (float*)vcache, nh, nkv, d, rot, page_size, interleaved, write_cache);
  else if (act_dtype == GG_BF16)
    gg_launch(rope_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, (__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, nkv, d, rot, page_size, interleaved, write_cache);
  else
    return gg_fail(GG_ERR_INVALID, "rope_kv_write: unknown dtype %d", act_dtype);
  return gg_check_launch("rope_kv_write");
}
