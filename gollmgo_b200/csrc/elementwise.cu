// Embedding gather, residual-add + RMSNorm, SiLU(gate)*up.
//
// The residual stream is float32 everywhere (the reference keeps it so:
// kernels/gollmgo_model.cu:46-61); the activations that feed matrix products
// are TA = float (true 32-bit path) or bfloat16 (serving path).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] = float(table[ids[t], :])   (reference: kernels/gollmgo_ops.cu:538-552,
// which leaves the row stale for an id out of range; here the row is zeroed and
// *bad_id is set, and the host has already refused such ids.)
// With token_src, token t comes from prev_tokens[token_src[t]] where token_src[t] >= 0: the
// token sampled on the device in the step before, which the host has not read yet.
template <typename TW>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                    float* __restrict__ out, int H, int V, int* bad_id,
                                    const int* __restrict__ token_src, const int* __restrict__ prev_tokens) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (token_src) {
    const int src = token_src[t];
    if (src >= 0) id = prev_tokens[src];
  }
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0 && bad_id) atomicExch(bad_id, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int gg_embed_gather(const int* ids, const void* table, int table_dtype, float* out,
                               int T, int H, int V, int* bad_id, const int* token_src,
                               const int* prev_tokens, cudaStream_t stream) {
  GG_REQUIRE(!token_src || prev_tokens, "embed_gather: token sources without the previous tokens");
  GG_REQUIRE(T >= 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
  if (T == 0) return GG_OK;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == GG_F32)
    gg_launch(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, ids, (const float*)table, out, H, V, bad_id, token_src, prev_tokens);
  else if (table_dtype == GG_BF16)
    gg_launch(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out, H, V, bad_id, token_src, prev_tokens);
  else
    return gg_fail(GG_ERR_INVALID, "embed_gather: unknown dtype %d", table_dtype);
  return gg_check_launch("embed_gather");
}

// ---------------------------------------------------------------- add + rmsnorm
// x = resid[r, :] (+ delta[r, :]);  if write_back: resid[r, :] = x;
// out[i, :] = TA( x * rsqrt(mean(x^2) + eps) * w )          r = rows ? rows[i] : i
// Formula: kernels/gollmgo_ops.cu:593-629; the residual add it is fused with is
// kernels/gollmgo_ops.cu:642-650.  Sum of squares, rsqrt and products in float32.
template <typename TA> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

// VEC: four elements per access (H a multiple of 4, rows 16-byte aligned).
template <typename TA, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const float* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int write_back) {
  extern __shared__ __align__(16) float xs[];          // H floats + 33 for the reduction
  float* red = xs + H;
  pdl_trigger();
  const int i = blockIdx.x;
  // the row list was copied in before the step began and the norm's weight never changes:
  // both are fetched while the kernel ahead is still finishing
  const int r = rows ? rows[i] : i;
  constexpr int PRE = 4;                               // float4 of the weight a thread keeps from before the wait
  float4 gpre[PRE];
  const bool pre = VEC && H <= PRE * 4 * (int)blockDim.x;
  if (pre) {
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
      const int c = (threadIdx.x + u * blockDim.x) * 4;
      gpre[u] = c < H ? *reinterpret_cast<const float4*>(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  float* xr = resid + (size_t)r * H;
  const TA* dr = delta ? delta + (size_t)r * H : nullptr;
  TA* o = out + (size_t)i * H;
  float ss = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      float4 x = *reinterpret_cast<const float4*>(xr + c);
      if (dr) {
        const float4 d = Vec4<TA>::load(dr + c);
        x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
        if (write_back) *reinterpret_cast<float4*>(xr + c) = x;
      }
      *reinterpret_cast<float4*>(xs + c) = x;
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float x = xr[c];
      if (dr) x += to_f32(dr[c]);
      xs[c] = x;
      if (write_back && dr) xr[c] = x;
      ss += x * x;
    }
  }
  const float total = block_sum(ss, red);
  const float rinv = rsqrtf(total / (float)H + eps);
  if (VEC && pre) {
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
      const int c = (threadIdx.x + u * blockDim.x) * 4;
      if (c < H) {
        const float4 x = *reinterpret_cast<const float4*>(xs + c);
        const float4 g = gpre[u];
        Vec4<TA>::store(o + c, make_float4(x.x * rinv * g.x, x.y * rinv * g.y, x.z * rinv * g.z, x.w * rinv * g.w));
      }
    }
  } else if (VEC) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      const float4 x = *reinterpret_cast<const float4*>(xs + c);
      const float4 g = *reinterpret_cast<const float4*>(w + c);
      Vec4<TA>::store(o + c, make_float4(x.x * rinv * g.x, x.y * rinv * g.y, x.z * rinv * g.z, x.w * rinv * g.w));
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f32<TA>(xs[c] * rinv * w[c]);
  }
}

template <typename TA>
static int launch_add_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                              const int* rows, int n, int H, float eps, int write_back,
                              cudaStream_t stream) {
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  GG_REQUIRE(smem <= 227 * 1024, "add_rmsnorm: width %d needs %zu B of shared memory (max 232448)", H, smem);
  const bool vec = H % 4 == 0 && ((size_t)resid % 16) == 0 && ((size_t)w % 16) == 0 &&
                   ((size_t)out % (4 * sizeof(TA))) == 0 && ((size_t)delta % (4 * sizeof(TA))) == 0;
  if (smem > 48 * 1024) {
    cudaError_t e = vec ? cudaFuncSetAttribute(add_rmsnorm_kernel<TA, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(add_rmsnorm_kernel<TA, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
  }
  if (vec) {
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    gg_launch(add_rmsnorm_kernel<TA, true>, dim3(n), dim3(threads), smem, stream, resid, (const TA*)delta, w, (TA*)out, rows, H, eps, write_back);
  } else {
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    gg_launch(add_rmsnorm_kernel<TA, false>, dim3(n), dim3(threads), smem, stream, resid, (const TA*)delta, w, (TA*)out, rows, H, eps, write_back);
  }
  return gg_check_launch("add_rmsnorm");
}

extern "C" int gg_add_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                              int act_dtype, const int* rows, int n, int H, float eps,
                              int write_back, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && H > 0 && eps > 0.f, "add_rmsnorm: bad sizes n=%d H=%d eps=%g", n, H, (double)eps);
  if (n == 0) return GG_OK;
  if (act_dtype == GG_F32) return launch_add_rmsnorm<float>(resid, delta, w, out, rows, n, H, eps, write_back, stream);
  if (act_dtype == GG_BF16) return launch_add_rmsnorm<__nv_bfloat16>(resid, delta, w, out, rows, n, H, eps, write_back, stream);
  return gg_fail(GG_ERR_INVALID, "add_rmsnorm: unknown dtype %d", act_dtype);
}

// ---------------------------------------------------------------- silu(gate) * up
// in: [T, 2*I] with gate in columns [0, I) and up in [I, 2I); out: [T, I]
// out = TA( g / (1 + exp(-g)) * u )     (kernels/gollmgo_ops.cu:361-374)
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ in, TA* __restrict__ out, int T, int I) {
  pdl_trigger();
  pdl_wait();
  const size_t n = (size_t)T * I;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t t = e / I;
    const int c = (int)(e - t * I);
    const float g = to_f32(in[t * 2 * I + c]);
    const float u = to_f32(in[t * 2 * I + I + c]);
    out[e] = from_f32<TA>(g / (1.f + expf(-g)) * u);
  }
}

// Four features per thread; grid (ceil(I/4/threads), T): no division per element.
template <typename TA>
__global__ void silu_mul_vec_kernel(const TA* __restrict__ in, TA* __restrict__ out, int I) {
  pdl_trigger();
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= I) return;
  const size_t t = blockIdx.y;
  const float4 g = Vec4<TA>::load(in + t * 2 * I + c);
  const float4 u = Vec4<TA>::load(in + t * 2 * I + I + c);
  float4 r;
  r.x = g.x / (1.f + expf(-g.x)) * u.x;
  r.y = g.y / (1.f + expf(-g.y)) * u.y;
  r.z = g.z / (1.f + expf(-g.z)) * u.z;
  r.w = g.w / (1.f + expf(-g.w)) * u.w;
  Vec4<TA>::store(out + t * I + c, r);
}

extern "C" int gg_silu_mul(const void* in, void* out, int act_dtype, int T, int I,
                           cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T, I);
  if (T == 0) return GG_OK;
  const size_t n = (size_t)T * I;
  const int threads = 256;
  if (I % 4 == 0 && T <= 65535 && ((size_t)in % 16) == 0 && ((size_t)out % 16) == 0) {
    dim3 grid((I / 4 + threads - 1) / threads, T);
    if (act_dtype == GG_F32) gg_launch(silu_mul_vec_kernel<float>, dim3(grid), dim3(threads), 0, stream, (const float*)in, (float*)out, I);
    else if (act_dtype == GG_BF16) gg_launch(silu_mul_vec_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, I);
    else return gg_fail(GG_ERR_INVALID, "silu_mul: unknown dtype %d", act_dtype);
    return gg_check_launch("silu_mul");
  }
  size_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act_dtype == GG_F32)
    gg_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, T, I);
  else if (act_dtype == GG_BF16)
    gg_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, T, I);
  else
    return gg_fail(GG_ERR_INVALID, "silu_mul: unknown dtype %d", act_dtype);
  return gg_check_launch("silu_mul");
}
