// Attention over the paged cache: the general kernels (any head size up to 256,
// any number of heads and groups, float32 or bfloat16 cache, optional window).
//
// One tile routine serves both shapes of work:
//   * a prompt portion: up to 16 consecutive query tokens of one sequence, one head;
//   * a decoded token:  up to 16 query heads that share one kv head, one token,
//     optionally over one slice of the context (split-KV), merged afterwards.
// It streams the keys and values of [lo, hi) through shared memory 64 tokens at a
// time and keeps a running maximum, sum and output per row (online softmax), all
// in float32.  Keys come only from the cache, found through the sequence's block
// table, so a portion sees every earlier portion and never another sequence.
//
// Formulas: kernels/gollmgo_paged_attn.cu:149-223 (scores, softmax, sum of p*V;
// kv head = head / (nh/nkv); scale = 1/sqrt(d)) and :234-384 (partition + merge).
// The reference's prompt kernel (kernels/gollmgo_ops.cu:377-446) reads only the
// current call's keys and masks by position alone; this one does not share those
// two properties.
#include "attention_common.cuh"
#include <stdlib.h>

#define ATT_BQ 16
#define ATT_BK 64
#define ATT_THREADS 128

template <typename TA, int DMAX>
__device__ __forceinline__ void attn_tile(const AttnArgs& a, int nrows, const TA* const* qptr_s,
                                          const int* pos_s, int kvh, const int* bt, int lo,
                                          int hi, float* smem, float* acc) {
  constexpr int NACC = ATT_BQ * DMAX / ATT_THREADS;
  const int d = a.d, ps = a.page_size;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* Qs = smem;                                  // [16][d]
  float* Ks = Qs + ATT_BQ * d;                       // [64][d+1]
  float* Vs = Ks + ATT_BK * (d + 1);                 // [64][d]
  float* Ss = Vs + ATT_BK * d;                       // [16][64]
  float* m_s = Ss + ATT_BQ * ATT_BK;                 // [16]
  float* l_s = m_s + ATT_BQ;                         // [16]
  float* al_s = l_s + ATT_BQ;                        // [16]
  const TA* kc = (const TA*)a.kcache;
  const TA* vc = (const TA*)a.vcache;

  for (int e = tid; e < ATT_BQ * d; e += ATT_THREADS) {
    const int r = e / d, c = e - r * d;
    Qs[e] = r < nrows ? to_f32(qptr_s[r][c]) : 0.f;
  }
  if (tid < ATT_BQ) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; al_s[tid] = 1.f; }
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  __syncthreads();

  const int kstart = (lo / ATT_BK) * ATT_BK;
  for (int kb = kstart; kb < hi; kb += ATT_BK) {
    // ---- stage keys and values of tokens [kb, kb+64)
    for (int j = warp; j < ATT_BK; j += ATT_THREADS / 32) {
      const int tok = kb + j;
      int page = -1;
      if (tok >= lo && tok < hi) page = bt[tok / ps];
      if (page >= 0) {
        const size_t base = (((size_t)page * a.nkv + kvh) * ps + (tok % ps)) * d;
        for (int c = lane; c < d; c += 32) {
          Ks[j * (d + 1) + c] = to_f32(kc[base + c]);
          Vs[j * d + c] = to_f32(vc[base + c]);
        }
      } else {
        for (int c = lane; c < d; c += 32) { Ks[j * (d + 1) + c] = 0.f; Vs[j * d + c] = 0.f; }
      }
    }
    __syncthreads();
    // ---- scores: thread (j = tid%64, rows tid/64 + 2i)
    {
      const int j = tid & 63, rb = tid >> 6;
      float s[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] = 0.f;
      const float* kr = Ks + j * (d + 1);
      for (int c = 0; c < d; ++c) {
        const float kv = kr[c];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = fmaf(Qs[(rb + 2 * i) * d + c], kv, s[i]);
      }
      const int tok = kb + j;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = rb + 2 * i;
        const int p = pos_s[r];
        const bool ok = tok >= lo && tok < hi && tok <= p && (a.window <= 0 || tok > p - a.window);
        Ss[r * ATT_BK + j] = ok ? s[i] * a.scale : -INFINITY;
      }
    }
    __syncthreads();
    // ---- running softmax: warp w owns rows 4w .. 4w+3
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp * 4 + i;
      const float s0 = Ss[r * ATT_BK + lane], s1 = Ss[r * ATT_BK + lane + 32];
      const float mx = warp_max(fmaxf(s0, s1));
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, mx);
      float p0 = 0.f, p1 = 0.f, alpha = 1.f;
      if (m_new != -INFINITY) {
        alpha = expf(m_old - m_new);
        p0 = expf(s0 - m_new);
        p1 = expf(s1 - m_new);
      }
      const float sum = warp_sum(p0 + p1);
      Ss[r * ATT_BK + lane] = p0;
      Ss[r * ATT_BK + lane + 32] = p1;
      if (lane == 0) { m_s[r] = m_new; l_s[r] = l_s[r] * alpha + sum; al_s[r] = alpha; }
    }
    __syncthreads();
    // ---- output: thread owns elements e = tid + 128*i of the [16][d] tile
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int e = tid + ATT_THREADS * i;
      if (e < ATT_BQ * d) {
        const int r = e / d, c = e - r * d;
        float o = acc[i] * al_s[r];
        const float* pr = Ss + r * ATT_BK;
        const float* vcol = Vs + c;
#pragma unroll 8
        for (int j = 0; j < ATT_BK; ++j) o = fmaf(pr[j], vcol[j * d], o);
        acc[i] = o;
      }
    }
    __syncthreads();
  }
}

template <int DMAX> __host__ __device__ constexpr int attn_smem_floats(int d) {
  return ATT_BQ * d + ATT_BK * (d + 1) + ATT_BK * d + ATT_BQ * ATT_BK + 3 * ATT_BQ;
}

// ---------------------------------------------------------------- prompt portions
template <typename TA, int DMAX>
__global__ void __launch_bounds__(ATT_THREADS) attn_prefill_kernel(AttnArgs a) {
  constexpr int NACC = ATT_BQ * DMAX / ATT_THREADS;
  extern __shared__ float smem[];
  __shared__ const TA* qptr_s[ATT_BQ];
  __shared__ int pos_s[ATT_BQ];
  pdl_wait();
  const int b = a.tile_seq[blockIdx.x], q0 = a.tile_q0[blockIdx.x];
  const int h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int t0 = a.cu_q_lens[b], qlen = a.cu_q_lens[b + 1] - t0;
  const int ctx = a.context_lens[b];
  const int qstart = ctx - qlen;                 // tokens cached before this step
  const int nrows = min(ATT_BQ, qlen - q0);
  if (threadIdx.x < ATT_BQ) {
    const int r = threadIdx.x;
    qptr_s[r] = r < nrows ? (const TA*)a.q + (size_t)(t0 + q0 + r) * a.q_stride + (size_t)h * a.d : nullptr;
    pos_s[r] = r < nrows ? qstart + q0 + r : -1;
  }
  __syncthreads();
  const int first = qstart + q0, last = first + nrows - 1;
  const int lo = a.window > 0 ? max(0, first - a.window + 1) : 0;
  float acc[NACC];
  attn_tile<TA, DMAX>(a, nrows, qptr_s, pos_s, kvh, a.block_tables + (size_t)b * a.bt_stride, lo, last + 1, smem, acc);
  pdl_trigger();
  const float* l_s = smem + ATT_BQ * a.d + ATT_BK * (a.d + 1) + ATT_BK * a.d + ATT_BQ * ATT_BK + ATT_BQ;
  TA* out = (TA*)a.out;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int e = threadIdx.x + ATT_THREADS * i;
    if (e < ATT_BQ * a.d) {
      const int r = e / a.d, c = e - r * a.d;
      if (r < nrows) out[(size_t)(t0 + q0 + r) * a.nh * a.d + (size_t)h * a.d + c] = from_f32<TA>(acc[i] / l_s[r]);
    }
  }
}

// ---------------------------------------------------------------- decoded tokens, split-KV
// grid (n_dec, nkv * ceil(G/16), num_splits).  Slice s of a context of n visible
// keys covers ceil(n/S) keys rounded up to 64.  Writes un-normalised partial
// outputs with their (max, sum); a slice without keys writes (-inf, 0).
template <typename TA, int DMAX>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(AttnArgs a) {
  constexpr int NACC = ATT_BQ * DMAX / ATT_THREADS;
  extern __shared__ float smem[];
  __shared__ const TA* qptr_s[ATT_BQ];
  __shared__ int pos_s[ATT_BQ];
  pdl_wait();
  const int G = a.nh / a.nkv, gchunks = (G + ATT_BQ - 1) / ATT_BQ;
  const int b = a.dec_seqs[blockIdx.x];
  const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * ATT_BQ;
  const int split = blockIdx.z, S = a.num_splits;
  const int nrows = min(ATT_BQ, G - g0);
  const int ctx = b >= 0 ? a.context_lens[b] : 0;      // b < 0: padding of a captured batch
  const int t = b >= 0 ? a.cu_q_lens[b] : 0;
  const int lo0 = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int n = ctx - lo0;
  int chunk = (n + S - 1) / S;
  chunk = ((chunk + ATT_BK - 1) / ATT_BK) * ATT_BK;
  const int lo = lo0 + split * chunk, hi = min(ctx, lo + chunk);
  if (threadIdx.x < ATT_BQ) {
    const int r = threadIdx.x;
    qptr_s[r] = r < nrows ? (const TA*)a.q + (size_t)t * a.q_stride + (size_t)(kvh * G + g0 + r) * a.d : nullptr;
    pos_s[r] = r < nrows ? ctx - 1 : -1;
  }
  __syncthreads();
  float acc[NACC];
  if (lo < hi) {
    attn_tile<TA, DMAX>(a, nrows, qptr_s, pos_s, kvh, a.block_tables + (size_t)b * a.bt_stride, lo, hi, smem, acc);
  } else {
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  }
  pdl_trigger();
  const float* m_s = smem + ATT_BQ * a.d + ATT_BK * (a.d + 1) + ATT_BK * a.d + ATT_BQ * ATT_BK;
  const float* l_s = m_s + ATT_BQ;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int e = threadIdx.x + ATT_THREADS * i;
    if (e < ATT_BQ * a.d) {
      const int r = e / a.d, c = e - r * a.d;
      if (r < nrows) {
        const size_t row = ((size_t)blockIdx.x * a.nh + kvh * G + g0 + r) * S + split;
        a.part_o[row * a.d + c] = acc[i];
        if (c == 0) {
          a.part_ml[row * 2] = lo < hi ? m_s[r] : -INFINITY;
          a.part_ml[row * 2 + 1] = lo < hi ? l_s[r] : 0.f;
        }
      }
    }
  }
}

// Merge of the slices: M = max m_s; o = sum_s e^{m_s-M} acc_s / sum_s e^{m_s-M} l_s
// (kernels/gollmgo_paged_attn.cu:331-384).  grid (n_dec, nh), one thread per column.
template <typename TA>
__global__ void attn_merge_kernel(AttnArgs a) {
  pdl_trigger();
  pdl_wait();
  const int b = a.dec_seqs[blockIdx.x];
  if (b < 0) return;
  const int h = blockIdx.y, S = a.num_splits, d = a.d;
  const int t = a.cu_q_lens[b];
  const size_t row0 = ((size_t)blockIdx.x * a.nh + h) * S;
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, a.part_ml[(row0 + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < S; ++s) {
    const float m = a.part_ml[(row0 + s) * 2];
    if (m != -INFINITY) L += expf(m - M) * a.part_ml[(row0 + s) * 2 + 1];
  }
  TA* out = (TA*)a.out + (size_t)t * a.nh * d + (size_t)h * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < S; ++s) {
      const float m = a.part_ml[(row0 + s) * 2];
      if (m != -INFINITY) o += expf(m - M) * a.part_o[(row0 + s) * d + c];
    }
    out[c] = from_f32<TA>(L > 0.f ? o / L : 0.f);
  }
}

// ---------------------------------------------------------------- launchers
static int check_common(const AttnArgs& a, const char* who) {
  GG_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "%s: %d heads are not a multiple of %d kv heads", who, a.nh, a.nkv);
  GG_REQUIRE(a.d > 0 && a.d <= 256, "%s: head size %d is outside 1..256", who, a.d);
  GG_REQUIRE(a.page_size > 0 && a.bt_stride > 0, "%s: bad page size %d or block table width %d", who, a.page_size, a.bt_stride);
  return GG_OK;
}

template <typename K> static int set_smem(K kernel, size_t bytes, const char* who) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  return GG_OK;
}

#define ATT_DISPATCH(KERNEL, grid, who)                                                        \
  do {                                                                                         \
    const size_t smem = (size_t)attn_smem_floats<0>(a.d) * sizeof(float);                      \
    int rc = GG_OK;                                                                            \
    if (dtype == GG_F32) {                                                                     \
      if (a.d <= 64) { rc = set_smem(KERNEL<float, 64>, smem, who); if (rc) return rc; gg_launch(KERNEL<float, 64>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
      else if (a.d <= 128) { rc = set_smem(KERNEL<float, 128>, smem, who); if (rc) return rc; gg_launch(KERNEL<float, 128>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
      else { rc = set_smem(KERNEL<float, 256>, smem, who); if (rc) return rc; gg_launch(KERNEL<float, 256>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
    } else if (dtype == GG_BF16) {                                                             \
      if (a.d <= 64) { rc = set_smem(KERNEL<__nv_bfloat16, 64>, smem, who); if (rc) return rc; gg_launch(KERNEL<__nv_bfloat16, 64>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
      else if (a.d <= 128) { rc = set_smem(KERNEL<__nv_bfloat16, 128>, smem, who); if (rc) return rc; gg_launch(KERNEL<__nv_bfloat16, 128>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
      else { rc = set_smem(KERNEL<__nv_bfloat16, 256>, smem, who); if (rc) return rc; gg_launch(KERNEL<__nv_bfloat16, 256>, dim3(grid), dim3(ATT_THREADS), smem, stream, a); } \
    } else {                                                                                   \
      return gg_fail(GG_ERR_INVALID, "%s: unknown dtype %d", who, dtype);                      \
    }                                                                                          \
  } while (0)

int attn_prefill_general(const AttnArgs& a, int dtype, int num_tiles, cudaStream_t stream) {
  GG_REQUIRE(num_tiles >= 0 && a.nh <= 65535, "attn_prefill: bad grid %d x %d", num_tiles, a.nh);
  if (num_tiles == 0) return GG_OK;
  dim3 grid(num_tiles, a.nh);
  ATT_DISPATCH(attn_prefill_kernel, grid, "attn_prefill");
  return gg_check_launch("attn_prefill");
}

int attn_decode_general(const AttnArgs& a, int dtype, int n_dec, cudaStream_t stream) {
  const int G = a.nh / a.nkv, gchunks = (G + ATT_BQ - 1) / ATT_BQ;
  GG_REQUIRE(a.nkv * gchunks <= 65535 && a.nh <= 65535, "attn_decode: too many heads");
  dim3 grid(n_dec, a.nkv * gchunks, a.num_splits);
  ATT_DISPATCH(attn_decode_kernel, grid, "attn_decode");
  return gg_check_launch("attn_decode");
}

int attn_merge_launch(const AttnArgs& a, int dtype, int n_dec, cudaStream_t stream) {
  dim3 mgrid(n_dec, a.nh);
  const int mthreads = a.d >= 128 ? 128 : (a.d >= 64 ? 64 : 32);
  if (dtype == GG_F32) gg_launch(attn_merge_kernel<float>, dim3(mgrid), dim3(mthreads), 0, stream, a);
  else gg_launch(attn_merge_kernel<__nv_bfloat16>, dim3(mgrid), dim3(mthreads), 0, stream, a);
  return gg_check_launch("attn_merge");
}

// Which tcgen05 prompt kernel a launch with allow_tc = 1 runs for a shape on this build and
// device: 3 = two heads per CTA in steps of 128 keys, 2 = the same in steps of 64, 1 = one head
// per CTA, 0 = none (the mma.sync or the general kernel).
extern "C" int gg_attn_prefill_choice(int dtype, int d, int page_size, int nh, int nkv) {
  static const bool wide = !(getenv("GOLLMGO_B200_ATTN_STEP") && atoi(getenv("GOLLMGO_B200_ATTN_STEP")) == 64);
  if (wide && attn_tc3_supported(dtype, d, page_size, nh, nkv)) return 3;
  if (attn_tc2_supported(dtype, d, page_size, nh, nkv)) return 2;
  return attn_tc_supported(dtype, d, page_size) ? 1 : 0;
}

// Three tile lists describe the same portions cut into 16, 64 and 128 query rows, for the
// general kernel, the mma.sync kernel and the tcgen05 kernel; the launcher picks the kernel
// from dtype, head size and what the caller allows.  T = rows of the q buffer, num_pages =
// pages of the cache, status = the word the tcgen05 kernel reports a timed-out wait in.
extern "C" int gg_attn_prefill(const void* q, long long q_stride, const void* kcache,
                               const void* vcache, int dtype, const int* block_tables,
                               int bt_stride, const int* cu_q_lens, const int* context_lens,
                               const int* tile_seq, const int* tile_q0, int num_tiles,
                               const int* tile64_seq, const int* tile64_q0, int num_tiles64,
                               const int* tile128_seq, const int* tile128_q0, int num_tiles128,
                               void* out, int T, int num_pages, int nh, int nkv, int d, int page_size,
                               int window, float scale, int allow_mma, int allow_tc, int* status,
                               cudaStream_t stream) {
  AttnArgs a = {};
  a.q = q; a.q_stride = q_stride; a.kcache = kcache; a.vcache = vcache;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_q_lens = cu_q_lens;
  a.context_lens = context_lens; a.out = out; a.nh = nh; a.nkv = nkv; a.d = d;
  a.page_size = page_size; a.window = window; a.scale = scale;
  int rc = check_common(a, "attn_prefill");
  if (rc) return rc;
  if (allow_tc && tile128_seq && status && q_stride % 8 == 0) {
    a.tile_seq = tile128_seq; a.tile_q0 = tile128_q0;
    // allow_tc: 1 = the best tcgen05 kernel for the shape, 2 = the one-head-per-CTA kernel only,
    // 3 = two heads per CTA in steps of 64 keys (what 1 gave before there were steps of 128)
    static const bool wide = !(getenv("GOLLMGO_B200_ATTN_STEP") && atoi(getenv("GOLLMGO_B200_ATTN_STEP")) == 64);
    if (allow_tc == 1 && wide && attn_tc3_supported(dtype, d, page_size, nh, nkv))
      return attn_prefill_tc3(a, num_tiles128, T, num_pages, status, stream);
    if (allow_tc != 2 && attn_tc2_supported(dtype, d, page_size, nh, nkv))
      return attn_prefill_tc2(a, num_tiles128, T, num_pages, status, stream);
    if (attn_tc_supported(dtype, d, page_size))
      return attn_prefill_tc(a, num_tiles128, T, num_pages, status, stream);
  }
  if (allow_mma && tile64_seq && attn_mma_supported(dtype, d) && q_stride % 8 == 0) {
    a.tile_seq = tile64_seq; a.tile_q0 = tile64_q0;
    return attn_prefill_mma(a, num_tiles64, stream);
  }
  a.tile_seq = tile_seq; a.tile_q0 = tile_q0;
  return attn_prefill_general(a, dtype, num_tiles, stream);
}

// Scratch the caller provides: part_o float[n_dec * nh * num_splits * d],
// part_ml float[n_dec * nh * num_splits * 2].
extern "C" int gg_attn_decode(const void* q, long long q_stride, const void* kcache,
                              const void* vcache, int dtype, const int* block_tables,
                              int bt_stride, const int* cu_q_lens, const int* context_lens,
                              const int* dec_seqs, int n_dec, int num_splits, float* part_o,
                              float* part_ml, void* out, int nh, int nkv, int d, int page_size,
                              int window, float scale, int allow_mma, cudaStream_t stream) {
  AttnArgs a = {};
  a.q = q; a.q_stride = q_stride; a.kcache = kcache; a.vcache = vcache;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_q_lens = cu_q_lens;
  a.context_lens = context_lens; a.out = out; a.nh = nh; a.nkv = nkv; a.d = d;
  a.page_size = page_size; a.window = window; a.scale = scale;
  a.dec_seqs = dec_seqs; a.num_splits = num_splits; a.part_o = part_o; a.part_ml = part_ml;
  int rc = check_common(a, "attn_decode");
  if (rc) return rc;
  GG_REQUIRE(n_dec >= 0 && num_splits >= 1 && num_splits <= 65535, "attn_decode: bad n_dec %d or splits %d", n_dec, num_splits);
  GG_REQUIRE(part_o && part_ml, "attn_decode: no scratch given");
  if (n_dec == 0) return GG_OK;
  bool merged = false;
  if (allow_mma && attn_mma_supported(dtype, d) && q_stride % 2 == 0)
    rc = attn_decode_mma(a, n_dec, stream, &merged);
  else
    rc = attn_decode_general(a, dtype, n_dec, stream);
  if (rc || merged) return rc;
  return attn_merge_launch(a, dtype, n_dec, stream);
}

// gg_attn_decode with the work of gg_rope_kv_write for the same tokens folded in: q is the raw
// projection output [T, (nh + 2 nkv) * d] (left as it is), the kernel rotates q and k with
// half-split pairs over the whole head and writes k and v into the cache at slot_mapping[t]
// (write_cache = 0: rotates q only).  bfloat16, head sizes 64 and 128, at most 16 heads per
// kv head; anything else is refused.
extern "C" int gg_attn_decode_rope(const void* qkv, long long q_stride, void* kcache, void* vcache, int dtype,
                                   const int* block_tables, int bt_stride, const int* cu_q_lens,
                                   const int* context_lens, const int* dec_seqs, int n_dec, int num_splits,
                                   float* part_o, float* part_ml, void* out, int nh, int nkv, int d,
                                   int page_size, int window, float scale, const int* positions,
                                   const int* slot_mapping, const double* inv_freq, int write_cache,
                                   cudaStream_t stream) {
  AttnArgs a = {};
  a.q = qkv; a.q_stride = q_stride; a.kcache = kcache; a.vcache = vcache;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_q_lens = cu_q_lens;
  a.context_lens = context_lens; a.out = out; a.nh = nh; a.nkv = nkv; a.d = d;
  a.page_size = page_size; a.window = window; a.scale = scale;
  a.dec_seqs = dec_seqs; a.num_splits = num_splits; a.part_o = part_o; a.part_ml = part_ml;
  a.rope_inv_freq = inv_freq; a.rope_positions = positions; a.slot_mapping = slot_mapping;
  a.rope_write_cache = write_cache;
  int rc = check_common(a, "attn_decode_rope");
  if (rc) return rc;
  GG_REQUIRE(n_dec >= 0 && num_splits >= 1 && num_splits <= 65535, "attn_decode_rope: bad n_dec %d or splits %d", n_dec, num_splits);
  GG_REQUIRE(part_o && part_ml, "attn_decode_rope: no scratch given");
  GG_REQUIRE(inv_freq != nullptr, "attn_decode_rope: no inverse frequencies given");
  GG_REQUIRE(attn_mma_supported(dtype, d), "attn_decode_rope: only bfloat16 with head size 64 or 128 (got dtype %d, head size %d)", dtype, d);
  if (n_dec == 0) return GG_OK;
  bool merged = false;
  rc = attn_decode_mma(a, n_dec, stream, &merged);
  if (rc || merged) return rc;
  return attn_merge_launch(a, dtype, n_dec, stream);
}

// Decode attention for large batches (bfloat16, head size 64 or 128): the work is cut into
// equal ranges of tiles instead of whole slices (attention_mma.cu).  Scratch the caller
// provides: pieces = n_dec * nkv * ceil((nh / nkv) / 16) + gg_attn_decode_flat_ctas(d);
// part_o float[pieces * 16 * d], part_ml float[pieces * 16 * 2], prefix int[prefix_ints] with
// prefix_ints >= n_dec + 1 + 2 * n_dec * nkv * ceil((nh / nkv) / 16).
extern "C" int gg_attn_decode_flat(const void* q, long long q_stride, const void* kcache, const void* vcache,
                                   int dtype, const int* block_tables, int bt_stride, const int* cu_q_lens,
                                   const int* context_lens, const int* dec_seqs, int n_dec, float* part_o,
                                   float* part_ml, int* prefix, int prefix_ints, void* out, int nh, int nkv, int d,
                                   int page_size, int window, float scale, cudaStream_t stream) {
  AttnArgs a = {};
  a.q = q; a.q_stride = q_stride; a.kcache = kcache; a.vcache = vcache;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_q_lens = cu_q_lens;
  a.context_lens = context_lens; a.out = out; a.nh = nh; a.nkv = nkv; a.d = d;
  a.page_size = page_size; a.window = window; a.scale = scale;
  a.dec_seqs = dec_seqs; a.num_splits = 0; a.part_o = part_o; a.part_ml = part_ml;
  int rc = check_common(a, "attn_decode_flat");
  if (rc) return rc;
  GG_REQUIRE(n_dec >= 0, "attn_decode_flat: bad n_dec %d", n_dec);
  GG_REQUIRE(part_o && part_ml && prefix, "attn_decode_flat: no scratch given");
  GG_REQUIRE(nkv > 0 && nh >= nkv && (long long)prefix_ints >= (long long)n_dec + 1 + 2LL * n_dec * nkv * ((nh / nkv + 15) / 16),
             "attn_decode_flat: prefix scratch of %d ints is too small for %d tokens", prefix_ints, n_dec);
  GG_REQUIRE(attn_mma_supported(dtype, d) && q_stride % 2 == 0,
             "attn_decode_flat: only bfloat16 with head size 64 or 128 (got dtype %d, head size %d)", dtype, d);
  if (n_dec == 0) return GG_OK;
  return attn_decode_flat(a, n_dec, prefix, stream);
}

extern "C" int gg_attn_decode_flat_ctas(int d) { return attn_decode_flat_ctas(d); }

// Clusters of `splits` decode CTAs that the device holds at once for head size d in
// bfloat16 with `group` query heads to a kv head; 0 where gg_attn_decode would not use
// clusters for that count.
extern "C" int gg_attn_decode_cluster_capacity(int dtype, int d, int splits, int group) {
  if (!attn_mma_supported(dtype, d)) return 0;
  return attn_decode_cluster_capacity(d, splits, group);
}
