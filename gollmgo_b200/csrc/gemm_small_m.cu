// Matrix products for a handful of tokens (decode): out[M, N] = x[M, K] W[N, K]^T with
// M <= 16, bfloat16 in, float32 accumulation.  At these sizes the product is a single
// pass over the weights, so the kernel is built to stream W from HBM at full rate:
//
//   * a CTA owns 16 rows of W (16 outputs) over the whole K; its 8 warps take
//     interleaved 64-wide spans of K and are summed through shared memory at the
//     end, in a fixed order (no atomics: the result does not depend on timing);
//   * the tensor cores are used "swapped": the 16 weight rows are the M side of
//     mma.sync m16n8k16 and the (up to 16) tokens the N side;
//   * a lane copies 16 contiguous bytes (8 values of k) of its two rows with
//     cp.async (bypassing L1) into a private shared-memory ring several iterations
//     ahead, and feeds each chunk to two MMAs.  Which physical k sits in
//     which k-slot of the instruction does not matter for a dot product, as long as
//     x uses the same placement, so no shuffles or shared-memory staging of W is
//     needed and every byte of W is read exactly once, coalesced.
//
// Epilogues: bfloat16 out; float32 out (LM head); SiLU-gated: rows 0-7 of the tile
// come from the gate weights and rows 8-15 from the up weights of the same 8
// features, and the CTA writes silu(gate) * up directly (the reference runs two
// products and an activation kernel: kernels/gollmgo_model.cu:746-768).
#include "attention_common.cuh"   // mma_bf16

#define GSM_WARPS 8
#define GSM_THREADS (GSM_WARPS * 32)
#define GSM_SPAN 64               // k per warp per iteration

enum { GSM_OUT_BF16 = 0, GSM_OUT_F32 = 1, GSM_OUT_SILU = 2, GSM_OUT_RESNORM = 3 };

// Two ways to keep an RMSNorm out of the chain of kernels (rms = sqrt(mean(h^2) + eps)):
//   * the product that ends a mixer or feed-forward (mode GSM_OUT_RESNORM) adds its result to
//     the float32 residual stream h in place, writes h * w (w the next norm's weight) in
//     bfloat16 where the norm's output would go, and leaves, per row tile and token, the
//     sum of h^2 over the tile's 16 columns in out_partials[tile * 16 + token];
//   * the product that follows takes that h * w as its x and multiplies row t of its result
//     by 1 / rms_t, which it gets from in_partials: the same as x = h * w / rms_t, since the
//     factor is one per token.  Sums run in a fixed order: no atomics, same result each run.
struct GsmFuse {
  const float* in_partials;   // [in_tiles, 16] sums of squares of this product's (unnormalised) x, or null
  int in_tiles;
  float inv_h, eps;           // 1 / hidden size, the norm's eps
  float* resid;               // GSM_OUT_RESNORM: [M, N] float32 residual stream, updated in place
  const float* norm_w;        // [N] weight of the norm that follows
  float* out_partials;        // [tiles of 16 columns, 16]
};

#define GSM_STAGES 6

// Rows of W (tile rows g and g+8) that a lane reads for row tile `tile`.
template <int MODE>
__device__ __forceinline__ void tile_rows(int tile, int g, int N, int& n_a, int& n_b) {
  if (MODE == GSM_OUT_SILU) {          // N = number of gated features I; W is [2I, K]: gate rows, then up rows
    n_a = tile * 8 + g;
    n_b = n_a < N ? N + n_a : -1;
    if (n_a >= N) n_a = -1;
  } else {
    n_a = tile * 16 + g;
    n_b = n_a + 8;
    if (n_a >= N) n_a = -1;
    if (n_b >= N) n_b = -1;
  }
}

// A CTA walks over row tiles blockIdx.x, blockIdx.x + gridDim.x, ... in groups of up to
// GROUP tiles.  Within a group the loop runs over K on the outside and the group's
// tiles on the inside, so a warp fetches its slice of x once per K step and uses it
// for every tile of the group.  Every lane keeps a private ring of GSM_STAGES x 64
// bytes in shared memory that cp.async fills ahead of use, across tile and group
// boundaries, so about five chunks of weights per lane (10 KB per warp) are in
// flight at any time; the lane that copies a chunk is the lane that consumes it, so
// waiting on its own copy groups is all the synchronisation the ring needs.
// GROUP x XB is the same for every shape, so the unrolled loop body keeps its size (a body
// several times larger measurably stalls on instruction fetch): CTAs with many row tiles
// share one fetch of x among GROUP tiles; CTAs with one or two tiles fetch the x chunks of
// XB K steps together instead, so that the latencies of those loads overlap.
template <int NT, int MODE, int GROUP, int XB>
__global__ void __launch_bounds__(GSM_THREADS)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                    const __nv_bfloat16* __restrict__ W, void* __restrict__ out, int M, int N, int K,
                    int num_tiles, const GsmFuse fuse) {
  __shared__ float row_scale[16];
  extern __shared__ __align__(16) unsigned char gsm_smem[];
  uint4* ring = reinterpret_cast<uint4*>(gsm_smem);                       // [warps][stages][4][32]
  float (*red)[16][8 * NT + 1] =
      reinterpret_cast<float (*)[16][8 * NT + 1]>(gsm_smem + (size_t)GSM_WARPS * GSM_STAGES * 4 * 32 * 16);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  const int iters = K > warp * GSM_SPAN ? (K - warp * GSM_SPAN + GSM_WARPS * GSM_SPAN - 1) / (GSM_WARPS * GSM_SPAN) : 0;
  const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const unsigned ring_base = smem_u32(ring) + (unsigned)((warp * GSM_STAGES * 4 * 32 + lane) * 16);

  // CTAs start at different places of K and wrap around, so that at any moment they ask L2
  // for different lines of x (every CTA reads all of x; in step they would all hit one line)
  const int rot = iters > 0 ? (int)(blockIdx.x % (unsigned)iters) : 0;
  // producer position: tile index within my tiles (group start + offset), k step, ring stage
  int p_g0 = 0, p_ki = 0, p_tj = 0, p_stage = 0;
  auto issue = [&]() {
    if (iters > 0 && p_g0 < my_tiles) {
      int n_a, n_b;
      tile_rows<MODE>(blockIdx.x + (p_g0 + p_tj) * gridDim.x, g, N, n_a, n_b);
      const int kk = p_ki + rot < iters ? p_ki + rot : p_ki + rot - iters;
      const int k0 = (kk * GSM_WARPS + warp) * GSM_SPAN + c * 8, k1 = k0 + 32;
      const unsigned dst = ring_base + (unsigned)(p_stage * 4 * 32 * 16);
      const __nv_bfloat16* wa = W + (size_t)max(n_a, 0) * K;
      const __nv_bfloat16* wb = W + (size_t)max(n_b, 0) * K;
      cp_async16(dst, wa + min(k0, K - 8), (n_a >= 0 && k0 < K) ? 16 : 0);
      cp_async16(dst + 512, wb + min(k0, K - 8), (n_b >= 0 && k0 < K) ? 16 : 0);
      cp_async16(dst + 1024, wa + min(k1, K - 8), (n_a >= 0 && k1 < K) ? 16 : 0);
      cp_async16(dst + 1536, wb + min(k1, K - 8), (n_b >= 0 && k1 < K) ? 16 : 0);
      const int gsize = min(GROUP, my_tiles - p_g0);
      if (++p_tj == gsize) {
        p_tj = 0;
        if (++p_ki == iters) { p_ki = 0; p_g0 += GROUP; }
      }
      p_stage = p_stage + 1 == GSM_STAGES ? 0 : p_stage + 1;
    }
    cp_async_commit();
  };

  const __nv_bfloat16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = g + 8 * j < M ? x + (size_t)(g + 8 * j) * ldx : nullptr;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // the weights are written by no kernel: start streaming them while the kernel before
  // this one is still finishing, then wait for it before touching x
#pragma unroll
  for (int s = 0; s < GSM_STAGES - 1; ++s) issue();
  pdl_trigger();
  pdl_wait();
  if (fuse.in_partials) {
    // 1 / rms of every token from the partial sums: thread (tl, tok) adds tiles tl, tl + 16, ...,
    // then thread tok adds the 16 results, in that order
    float (*sc)[17] = reinterpret_cast<float (*)[17]>(&red[0][0][0]);
    const int tl = threadIdx.x >> 4, tok = threadIdx.x & 15;
    float v = 0.f;
    for (int tile = tl; tile < fuse.in_tiles; tile += GSM_THREADS / 16) v += fuse.in_partials[tile * 16 + tok];
    sc[tl][tok] = v;
    __syncthreads();
    if (threadIdx.x < 16) {
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < GSM_THREADS / 16; ++i) sum += sc[i][threadIdx.x];
      row_scale[threadIdx.x] = rsqrtf(sum * fuse.inv_h + fuse.eps);
    }
    __syncthreads();
  }
  int c_stage = 0;
  for (int g0 = 0; g0 < my_tiles; g0 += GROUP) {
    const int gsize = min(GROUP, my_tiles - g0);
    float acc[GROUP][NT][4];
#pragma unroll
    for (int t = 0; t < GROUP; ++t)
#pragma unroll
      for (int j = 0; j < NT; ++j) { acc[t][j][0] = acc[t][j][1] = acc[t][j][2] = acc[t][j][3] = 0.f; }
    // x comes from L2 and a K step is short: a lane asks for its chunks of XB steps at once,
    // so that their latencies overlap
    for (int kb = 0; kb < iters; kb += XB) {
      uint4 xb[XB][2 * NT];
#pragma unroll
      for (int u = 0; u < XB; ++u) {
        const int ki = kb + u;
        const int kk = ki + rot < iters ? ki + rot : ki + rot - iters;
        const int k0 = (kk * GSM_WARPS + warp) * GSM_SPAN + c * 8, k1 = k0 + 32;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          xb[u][2 * j] = (xr[j] && ki < iters && k0 < K) ? __ldg(reinterpret_cast<const uint4*>(xr[j] + k0)) : zero;
          xb[u][2 * j + 1] = (xr[j] && ki < iters && k1 < K) ? __ldg(reinterpret_cast<const uint4*>(xr[j] + k1)) : zero;
        }
      }
#pragma unroll
      for (int u = 0; u < XB; ++u) {
        if (kb + u < iters) {
#pragma unroll
          for (int t = 0; t < GROUP; ++t) {
            if (t < gsize) {
              issue();
              cp_async_wait<GSM_STAGES - 1>();
              const uint4* st = ring + ((size_t)(warp * GSM_STAGES + c_stage) * 4) * 32 + lane;
              const uint4 w0 = st[0], w1 = st[32], w2 = st[64], w3 = st[96];
              c_stage = c_stage + 1 == GSM_STAGES ? 0 : c_stage + 1;
#pragma unroll
              for (int j = 0; j < NT; ++j) {
                const uint4 x0 = xb[u][2 * j], x1 = xb[u][2 * j + 1];
                unsigned a[4];
                a[0] = w0.x; a[1] = w1.x; a[2] = w0.y; a[3] = w1.y;
                mma_bf16(acc[t][j], a, x0.x, x0.y);
                a[0] = w0.z; a[1] = w1.z; a[2] = w0.w; a[3] = w1.w;
                mma_bf16(acc[t][j], a, x0.z, x0.w);
                a[0] = w2.x; a[1] = w3.x; a[2] = w2.y; a[3] = w3.y;
                mma_bf16(acc[t][j], a, x1.x, x1.y);
                a[0] = w2.z; a[1] = w3.z; a[2] = w2.w; a[3] = w3.w;
                mma_bf16(acc[t][j], a, x1.z, x1.w);
              }
            }
          }
        }
      }
    }
    // per tile of the group: sum the 8 warps through shared memory, then the epilogue
#pragma unroll
    for (int t = 0; t < GROUP; ++t) {
      if (t < gsize) {
        // accumulators: [0],[1] = (row g, tokens 2c, 2c+1), [2],[3] = (row g+8, same tokens)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          red[warp][g][8 * j + 2 * c] = acc[t][j][0];
          red[warp][g][8 * j + 2 * c + 1] = acc[t][j][1];
          red[warp][g + 8][8 * j + 2 * c] = acc[t][j][2];
          red[warp][g + 8][8 * j + 2 * c + 1] = acc[t][j][3];
        }
        __syncthreads();
        const int tile = blockIdx.x + (g0 + t) * gridDim.x;
        if (MODE == GSM_OUT_SILU) {
          // thread -> (token, feature r of 8): contiguous features per token
          for (int e = threadIdx.x; e < 8 * NT * 8; e += GSM_THREADS) {
            const int tok = e >> 3, r = e & 7;
            const int f = tile * 8 + r;
            if (tok < M && f < N) {
              float gate = 0.f, up = 0.f;
#pragma unroll
              for (int wv = 0; wv < GSM_WARPS; ++wv) { gate += red[wv][r][tok]; up += red[wv][r + 8][tok]; }
              if (fuse.in_partials) { gate *= row_scale[tok]; up *= row_scale[tok]; }
              const float v = gate / (1.f + expf(-gate)) * up;
              reinterpret_cast<__nv_bfloat16*>(out)[(size_t)tok * N + f] = __float2bfloat16_rn(v);
            }
          }
        } else if (MODE == GSM_OUT_RESNORM) {
          // 16 neighbouring lanes hold the 16 columns of one token
          for (int e = threadIdx.x; e < 8 * NT * 16; e += GSM_THREADS) {
            const int tok = e >> 4, r = e & 15;
            const int n = tile * 16 + r;
            float h = 0.f;
            if (tok < M && n < N) {
              float v = 0.f;
#pragma unroll
              for (int wv = 0; wv < GSM_WARPS; ++wv) v += red[wv][r][tok];
              if (fuse.in_partials) v *= row_scale[tok];
              h = fuse.resid[(size_t)tok * N + n] + v;
              fuse.resid[(size_t)tok * N + n] = h;
              reinterpret_cast<__nv_bfloat16*>(out)[(size_t)tok * N + n] = __float2bfloat16_rn(h * fuse.norm_w[n]);
            }
            float sq = h * h;
            sq += __shfl_xor_sync(0xffffffffu, sq, 8);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            if (r == 0) fuse.out_partials[tile * 16 + tok] = sq;
          }
        } else {
          for (int e = threadIdx.x; e < 8 * NT * 16; e += GSM_THREADS) {
            const int tok = e >> 4, r = e & 15;
            const int n = tile * 16 + r;
            if (tok < M && n < N) {
              float v = 0.f;
#pragma unroll
              for (int wv = 0; wv < GSM_WARPS; ++wv) v += red[wv][r][tok];
              if (fuse.in_partials) v *= row_scale[tok];
              if (MODE == GSM_OUT_F32) reinterpret_cast<float*>(out)[(size_t)tok * N + n] = v;
              else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)tok * N + n] = __float2bfloat16_rn(v);
            }
          }
        }
        __syncthreads();
      }
    }
  }
  cp_async_wait<0>();
}

// mode: 0 = bfloat16 out [M, N]; 1 = float32 out [M, N]; 2 = W is [2N, K] (gate rows then
// up rows) and out is bfloat16 [M, N] = silu(x Wg^T) * (x Wu^T); 3 = out is the bfloat16
// input of the next norm and resid / norm_w / out_partials are used (see GsmFuse).
// in_partials (or null) with in_tiles, hidden and eps: x is an unnormalised norm input.
extern "C" int gg_gemm_small_m_fused(const void* x, long long ldx, const void* W, void* out, int M, int N,
                                     int K, int mode, const float* in_partials, int in_tiles, int hidden,
                                     float eps, float* resid, const float* norm_w, float* out_partials,
                                     cudaStream_t stream) {
  GG_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_small_m: bad sizes M=%d N=%d K=%d", M, N, K);
  GG_REQUIRE(M <= 16, "gemm_small_m: %d tokens; this kernel takes at most 16", M);
  GG_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_small_m: K=%d and the row stride %lld of x must be multiples of 8", K, ldx);
  GG_REQUIRE(((size_t)x % 16) == 0 && ((size_t)W % 16) == 0, "gemm_small_m: x and W must be 16-byte aligned");
  GG_REQUIRE(mode >= 0 && mode <= 3, "gemm_small_m: unknown mode %d", mode);
  GG_REQUIRE(!in_partials || (in_tiles > 0 && hidden > 0), "gemm_small_m: partial sums without their sizes");
  GG_REQUIRE(mode != GSM_OUT_RESNORM || (resid && norm_w && out_partials), "gemm_small_m: mode 3 needs resid, norm_w and out_partials");
  if (M == 0) return GG_OK;
  GsmFuse fuse = {};
  fuse.in_partials = in_partials; fuse.in_tiles = in_tiles;
  fuse.inv_h = hidden > 0 ? 1.0f / (float)hidden : 0.f; fuse.eps = eps;
  fuse.resid = resid; fuse.norm_w = norm_w; fuse.out_partials = out_partials;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)W;
  const int num_tiles = mode == GSM_OUT_SILU ? (N + 7) / 8 : (N + 15) / 16;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  const int grid = num_tiles < 2 * num_sms ? num_tiles : 2 * num_sms;
  const size_t ring_bytes = (size_t)GSM_WARPS * GSM_STAGES * 4 * 32 * 16;
#define GSM_LAUNCH(NT, MODE, GROUP, XB)                                                               \
  do {                                                                                                \
    const size_t smem = ring_bytes + sizeof(float) * GSM_WARPS * 16 * (8 * NT + 1);                   \
    static bool set = false;                                                                          \
    if (!set) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(gemm_small_m_kernel<NT, MODE, GROUP, XB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_small_m: %s", cudaGetErrorString(e));   \
      set = true;                                                                                     \
    }                                                                                                 \
    gg_launch(gemm_small_m_kernel<NT, MODE, GROUP, XB>, dim3(grid), dim3(GSM_THREADS), smem, stream, xp, ldx, wp, out, M, N, K, num_tiles, fuse); \
  } while (0)
#define GSM_MODES(NT, GROUP, XB)                                       \
  do {                                                                 \
    if (mode == 0) GSM_LAUNCH(NT, GSM_OUT_BF16, GROUP, XB);            \
    else if (mode == 1) GSM_LAUNCH(NT, GSM_OUT_F32, GROUP, XB);        \
    else if (mode == 2) GSM_LAUNCH(NT, GSM_OUT_SILU, GROUP, XB);       \
    else GSM_LAUNCH(NT, GSM_OUT_RESNORM, GROUP, XB);                   \
  } while (0)
  const int per_cta = (num_tiles + grid - 1) / grid;      // most row tiles one CTA gets
  if (M <= 8) {
    if (per_cta == 1) GSM_MODES(1, 1, 8); else if (per_cta == 2) GSM_MODES(1, 2, 4); else GSM_MODES(1, 8, 1);
  } else {
    if (per_cta == 1) GSM_MODES(2, 1, 4); else if (per_cta == 2) GSM_MODES(2, 2, 2); else GSM_MODES(2, 4, 1);
  }
#undef GSM_MODES
#undef GSM_LAUNCH
  return gg_check_launch("gemm_small_m");
}

extern "C" int gg_gemm_small_m(const void* x, long long ldx, const void* W, void* out, int M, int N,
                               int K, int mode, cudaStream_t stream) {
  GG_REQUIRE(mode >= 0 && mode <= 2, "gemm_small_m: unknown mode %d", mode);
  return gg_gemm_small_m_fused(x, ldx, W, out, M, N, K, mode, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr, stream);
}
