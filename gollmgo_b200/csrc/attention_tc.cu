// Causal attention of prompt portions on tcgen05, bfloat16, head sizes 64 and 128.
//
// Same contract as the other prompt kernels (attention.cu, attention_mma.cu): keys and
// values come only from the paged cache through the sequence's block table, masking is by
// absolute position (and an optional window), kv head = head / (nh/nkv), scale 1/sqrt(d).
//
// One CTA takes 128 query rows of one head and walks over the keys 128 at a time:
//   warp 0   drives TMA: the Q tile once (two 64-column boxes of the qkv buffer), then
//            per step the K and V tiles, lane p fetching page p as one box of
//            [64 columns x page] per half, from a 4-d tensor map over the cache
//            [pages, kv heads, page size, d].  A page that is not there (beyond the
//            context, or given back behind a window) is asked for at a page index past
//            the end, which TMA fills with zeros.  Two stages each for K and V.
//   warp 1   one lane issues the MMAs: S = Q K^T (128 x 128 x 128, K-major operands)
//            into one of two score buffers in tensor memory, and O += P V with V as an
//            MN-major operand straight from its [key][d] layout.  The product for the
//            next scores is issued before this step's P V, so the tensor core works on
//            it while the softmax warps are busy.
//   warps 2-9  softmax: two threads per query row (row = tensor-memory lane; each takes
//            64 of a step's 128 keys and half of O's columns), so row maxima and sums
//            need no shuffles, only one exchange per step.  A thread's 64 scores are read
//            once with tcgen05.ld and kept in registers, exponentials are
//            base 2 against a running reference maximum that is only moved (and O
//            rescaled through tcgen05.ld/st) when a row's maximum has grown by more than
//            2^8; P goes to shared memory in the swizzled K-major layout the second
//            product reads.  At the end O is divided by the row sums and stored.
// Tensor memory: columns [0,128) and [128,256) scores, [256,384) O.
// All waits are bounded; a wait that runs out sets *status and the CTA winds down.
#include "attention_common.cuh"
#include "tc_common.cuh"
// fast_exp2 comes with attention_common.cuh

#define ATC_BQ 128
#define ATC_BK 128
#define ATC_THREADS 320                     // TMA warp, MMA warp, eight softmax warps
#define ATC_SOFTMAX_THREADS 256
#define ATC_HALF_BYTES (128 * 64 * 2)       // [128 rows x 64 columns] bf16: rows of 128 bytes, swizzled
#define ATC_P_BYTES (2 * ATC_HALF_BYTES)    // P: 128 rows x 128 keys
#define ATC_LOG2E 1.4426950408889634f

enum { ATC_ERR_PRODUCER = 11, ATC_ERR_MMA = 12, ATC_ERR_SOFTMAX = 13 };

// Barrier over the 256 softmax threads only (named barrier 1), and the same with a vote:
// true only if every thread passes true.  Every softmax thread reaches these in the same
// order whatever its waits returned, so nobody is left behind at one.
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool softmax_all(bool mine) {
  unsigned out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 256, q;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(out) : "r"((unsigned)mine) : "memory");
  return out != 0;
}

struct AtcArgs {
  AttnArgs a;
  int num_pages;          // pages in the cache (an index >= this is filled with zeros)
  int* status;
};

// A Q, K or V tile is [128 rows x D]: D/64 halves.
template <int D>
__global__ void __launch_bounds__(ATC_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const AtcArgs args) {
  extern __shared__ unsigned char atc_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[16];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  __shared__ float xchg[2][2][ATC_BQ];       // [step parity][half][row]: row maxima of the two halves
  __shared__ float xsum[2][ATC_BQ];
  constexpr int ATC_D = D;
  constexpr int HALVES = D / 64;
  constexpr unsigned ATC_TILE_BYTES = HALVES * ATC_HALF_BYTES;
  const AttnArgs& a = args.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned base = (tc_smem(atc_smem_raw) + 1023u) & ~1023u;
  const unsigned q_smem = base, k_smem = base + ATC_TILE_BYTES, v_smem = k_smem + 2 * ATC_TILE_BYTES,
                 p_smem = v_smem + 2 * ATC_TILE_BYTES;
  const unsigned q_full = tc_smem(&bars[0]), k_full0 = tc_smem(&bars[1]), k_empty0 = tc_smem(&bars[3]),
                 v_full0 = tc_smem(&bars[5]), v_empty0 = tc_smem(&bars[7]), s_full0 = tc_smem(&bars[9]),
                 s_empty0 = tc_smem(&bars[11]), p_full = tc_smem(&bars[13]), pv_done = tc_smem(&bars[14]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1);
      mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1);
      mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 8);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_base_s;
  pdl_trigger();

  // ---- what this CTA works on (lists copied in before the step began: read before the wait)
  // grid (heads, tiles): the heads of one tile are neighbours, and the caller lists the tiles
  // with the most keys first, so the long ones start early and the short ones fill the end
  const int b = a.tile_seq[blockIdx.y], q0 = a.tile_q0[blockIdx.y];
  const int h = blockIdx.x, kvh = h / (a.nh / a.nkv);
  const int t0 = a.cu_q_lens[b], qlen = a.cu_q_lens[b + 1] - t0;
  const int ctx = a.context_lens[b];
  const int qstart = ctx - qlen;
  const int nrows = min(ATC_BQ, qlen - q0);
  const int first = qstart + q0;                       // position of the tile's first query
  const int hi = first + nrows;
  const int lo = a.window > 0 ? max(0, first - a.window + 1) : 0;
  const int kstart = (lo / ATC_BK) * ATC_BK;
  const int ntiles = (hi - kstart + ATC_BK - 1) / ATC_BK;
  const int ps = a.page_size, pages_per_tile = ATC_BK / ps;
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer: the whole warp; lane p fetches page p of a tile (two
    // boxes, one per half of d), first for the keys, then for the values, so the block
    // table look-ups and the issue of the many small copies run side by side
    const int* bt = a.block_tables + (size_t)b * a.bt_stride;
    if (lane == 0) {
      mbar_expect_tx(q_full, ATC_TILE_BYTES);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf)
        tma_load_2d(q_smem + hf * ATC_HALF_BYTES, &map_q, h * ATC_D + hf * 64, t0 + q0, q_full);
    }
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j & 1;
      const unsigned phase = (j >> 1) & 1;
      const int kb = kstart + j * ATC_BK;
      int page = -1;
      if (lane < pages_per_tile) {
        const int tok = kb + lane * ps;
        if (tok < hi && tok + ps > lo) page = __ldg(bt + tok / ps);
        if (page < 0) page = args.num_pages;                   // past the end: TMA fills zeros
      }
      const unsigned row_off = (unsigned)(lane * ps * 128);
      for (int which = 0; which < 2 && ok; ++which) {          // keys, then values
        const unsigned full = (which ? v_full0 : k_full0) + 8 * s, empty = (which ? v_empty0 : k_empty0) + 8 * s;
        const unsigned dst = (which ? v_smem : k_smem) + s * ATC_TILE_BYTES;
        const CUtensorMap* map = which ? &map_v : &map_k;
        ok = mbar_wait(empty, phase ^ 1) && !*(volatile int*)&abort_s;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(full, ATC_TILE_BYTES);
        __syncwarp();
        if (lane < pages_per_tile) {
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf)
            tma_load_4d(dst + hf * ATC_HALF_BYTES + row_off, map, hf * 64, 0, kvh, page, full);
        }
      }
    }
    if (!ok && lane == 0) { atomicExch(args.status, ATC_ERR_PRODUCER); atomicExch(&abort_s, 1); }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    // instruction descriptors: f32 accumulate, bf16 inputs, M = 128; scores: N = 128 keys
    const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    // O += P V: N = D, B (V) is MN-major
    const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (((unsigned)D >> 3) << 17) | ((128u >> 4) << 24);
    const unsigned tmem_o = tmem_base + 256;
    bool ok = mbar_wait(q_full, 0);
    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1;
      const unsigned phase = (j >> 1) & 1;
      if (!mbar_wait(k_full0 + 8 * s, phase)) return false;
      if (!mbar_wait(s_empty0 + 8 * s, phase ^ 1)) return false;
      tc_fence_after();
      const unsigned kt = k_smem + s * ATC_TILE_BYTES;
#pragma unroll
      for (int k = 0; k < ATC_D / 16; ++k) {
        const unsigned off = (k >> 2) * ATC_HALF_BYTES + (k & 3) * 32;
        tc_mma(tmem_base + s * 128, tc_smem_desc_lbo(q_smem + off, 1, 64), tc_smem_desc_lbo(kt + off, 1, 64),
               idesc_qk, k > 0 ? 1u : 0u);
      }
      tc_commit(s_full0 + 8 * s);          // scores ready
      tc_commit(k_empty0 + 8 * s);         // key tile free
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < ntiles && ok; ++j) {
      if (*(volatile int*)&abort_s) { ok = false; break; }
      if (j + 1 < ntiles) ok = issue_qk(j + 1);
      if (!ok) break;
      const int s = j & 1;
      if (!mbar_wait(p_full, j & 1)) { ok = false; break; }
      if (!mbar_wait(v_full0 + 8 * s, (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      const unsigned vt = v_smem + s * ATC_TILE_BYTES;
#pragma unroll
      for (int k = 0; k < ATC_BK / 16; ++k) {
        // A = P (K-major: keys contiguous), 16 keys = 32 bytes within a half of 64 keys
        const unsigned p_off = (k >> 2) * ATC_HALF_BYTES + (k & 3) * 32;
        // B = V (MN-major: d contiguous): 16 keys further = 16 rows of 128 bytes; the second
        // half of d is one half tile (LBO) further; groups of 8 keys are 1024 bytes apart (SBO)
        tc_mma(tmem_o, tc_smem_desc_lbo(p_smem + p_off, 1, 64),
               tc_smem_desc_lbo(vt + k * 16 * 128, ATC_HALF_BYTES >> 4, 64), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
      }
      tc_commit(pv_done);                  // O holds this step; P may be overwritten
      tc_commit(v_empty0 + 8 * s);
    }
    if (!ok) { atomicExch(args.status, ATC_ERR_MMA); atomicExch(&abort_s, 1); }
  } else if (warp >= 2) {
    // ---------------- softmax and epilogue: two threads per query row.  Warps 2-5 take the
    // first 64 keys of a step (and the first half of O's columns), warps 6-9 the second; a
    // warp reads the tensor-memory lanes of its quarter (warp % 4).  The two threads of a row
    // exchange their maxima through shared memory once per step and their sums at the end.
    const int quarter = warp & 3, sub = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int pos = first + r;
    const bool row_ok = r < nrows;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    constexpr int OC = D / 2;                             // O columns of this thread
    const unsigned tmem_o = lane_addr + 256 + sub * OC;
    const float sc = a.scale * ATC_LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    const int stale_hi = (hi + ps - 1) / ps * ps;        // end of the last page that is fetched
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
      const int kb = kstart + j * ATC_BK + sub * 64;      // first key of this thread's 64
      ok = softmax_all(mbar_wait(s_full0 + 8 * s, (j >> 1) & 1) && !*(volatile int*)&abort_s);
      if (!ok) break;
      tc_fence_after();
      const unsigned tmem_s = lane_addr + s * 128 + sub * 64;
      const bool interior = kb >= lo && kb + 63 <= first && (a.window <= 0 || kb > first + nrows - 1 - a.window);
      // the row's 64 scores, once, into registers (scaled to base 2; masked ones -inf)
      float sv[64];
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        unsigned v[32];
        tc_load32(tmem_s + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[c + i] = __uint_as_float(v[i]) * sc;
      }
      // the scores are in registers: the buffer can take the scores after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty0 + 8 * s);
      if (!interior) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int tk = kb + i;
          const bool keep = row_ok && tk >= lo && tk <= pos && (a.window <= 0 || tk > pos - a.window);
          if (!keep) sv[i] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i) mx = fmaxf(mx, sv[i]);
      xchg[j & 1][sub][r] = mx;
      softmax_sync();
      mx = fmaxf(mx, xchg[j & 1][sub ^ 1][r]);
      // move the reference maximum only when some row of the warp has outgrown it by 2^8
      const bool grow = mx > m_ref + 8.f;
      const bool rescale = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (rescale) {
        const float m_new = fmaxf(m_ref, mx);
        alpha = m_new == -INFINITY ? 1.f : exp2f(m_ref - m_new);       // m_ref = -inf gives 0
        m_ref = m_new;
        l *= alpha;
      }
      if (j > 0) {
        // the product of the step before must be complete: it read P, and it wrote O
        ok = softmax_all(mbar_wait(pv_done, (j - 1) & 1));
        if (!ok) break;
        tc_fence_after();
        if (rescale) {
#pragma unroll
          for (int c = 0; c < OC; c += 32) {
            unsigned v[32];
            tc_load32(tmem_o + c, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tc_store32(tmem_o + c, v);
          }
          tc_wait_store();
        }
      }
      // The last page of the last tile may hold rows past the context: whatever the page's
      // owner before left there.  Their P is zero, but zero times a NaN or an infinity is not:
      // those rows of V are cleared before the product reads them (the product waits for
      // every softmax warp's arrival on p_full).
      if (j == ntiles - 1 && stale_hi > ctx) {
        ok = softmax_all(mbar_wait(v_full0 + 8 * s, (j >> 1) & 1) && !*(volatile int*)&abort_s);
        if (!ok) break;
        const int tile0 = kstart + j * ATC_BK;
        const int z0 = max(ctx, tile0) - tile0, z1 = min(stale_hi, tile0 + ATC_BK) - tile0;
        if (r >= z0 && r < z1) {
          for (int hf = sub; hf < D / 64; hf += 2) {
            const unsigned row = v_smem + s * ATC_TILE_BYTES + hf * ATC_HALF_BYTES + (unsigned)r * 128;
#pragma unroll
            for (int c = 0; c < 128; c += 16)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(row + c), "r"(0u) : "memory");
          }
        }
      }
      // p = 2^(s - m_ref), row sum, P to shared memory (bf16, swizzled K-major): this thread's
      // 64 keys are half `sub` of the P tile
      const float mr = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        unsigned pk[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float p0 = fast_exp2(sv[c + i] - mr), p1 = fast_exp2(sv[c + i + 1] - mr);   // 2^-inf = 0
          sum += p0 + p1;
          __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
          pk[i >> 1] = *reinterpret_cast<unsigned*>(&t);
        }
        const unsigned addr = p_smem + sub * ATC_HALF_BYTES + (unsigned)r * 128 + (unsigned)(((c >> 3) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                     "r"(pk[3]) : "memory");
      }
      l += sum;
      fence_async_smem();                  // P is read by the tensor core (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && ntiles > 0) ok = softmax_all(mbar_wait(pv_done, (ntiles - 1) & 1));
    if (!ok) { atomicExch(args.status, ATC_ERR_SOFTMAX); atomicExch(&abort_s, 1); }
    // the row's sum is the two threads' sums (both used the same reference maxima)
    xsum[sub][r] = l;
    softmax_sync();
    l += xsum[sub ^ 1][r];
    tc_fence_after();
    if (ok && !*(volatile int*)&abort_s) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)(t0 + q0 + r) * a.nh * ATC_D + (size_t)h * ATC_D + sub * OC;
#pragma unroll
      for (int c = 0; c < OC; c += 32) {
        unsigned v[32];
        tc_load32(tmem_o + c, v);
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 pk;
            __nv_bfloat162 t0v = __floats2bfloat162_rn(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            __nv_bfloat162 t1v = __floats2bfloat162_rn(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            __nv_bfloat162 t2v = __floats2bfloat162_rn(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            __nv_bfloat162 t3v = __floats2bfloat162_rn(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            pk.x = *reinterpret_cast<unsigned*>(&t0v); pk.y = *reinterpret_cast<unsigned*>(&t1v);
            pk.z = *reinterpret_cast<unsigned*>(&t2v); pk.w = *reinterpret_cast<unsigned*>(&t3v);
            *reinterpret_cast<uint4*>(o + c + i) = pk;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------- host side
bool attn_tc_supported(int dtype, int d, int page_size) {
  return dtype == GG_BF16 && (d == 64 || d == 128) && page_size >= 8 && page_size <= 128 && (page_size & (page_size - 1)) == 0;
}

static int encode(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box) {
  GgEncodeTiledFn fn = gg_encode_tiled();
  if (!fn) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc: the driver has no cuTensorMapEncodeTiled");
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return GG_OK;
}

// a.tile_seq / a.tile_q0 list tiles of 128 query rows.  T = rows of the q buffer.
int attn_prefill_tc(const AttnArgs& a, int num_tiles, int T, int num_pages, int* status, cudaStream_t stream) {
  GG_REQUIRE(num_tiles >= 0 && num_tiles <= 65535, "attn_prefill_tc: %d tiles in one launch", num_tiles);
  GG_REQUIRE(status != nullptr, "attn_prefill_tc: no status word given");
  GG_REQUIRE(a.q_stride % 8 == 0 && ((size_t)a.q % 16) == 0, "attn_prefill_tc: q rows must be 16-byte aligned");
  if (num_tiles == 0) return GG_OK;
  CUtensorMap map_q, map_k, map_v;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a.nh * a.d, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)a.q_stride * 2};
    cuuint32_t box[2] = {64, ATC_BQ};
    int rc = encode(&map_q, a.q, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t D = (cuuint64_t)a.d;
    cuuint64_t dims[4] = {D, (cuuint64_t)a.page_size, (cuuint64_t)a.nkv, (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {D * 2, (cuuint64_t)a.page_size * D * 2, (cuuint64_t)a.nkv * a.page_size * D * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)a.page_size, 1, 1};
    int rc = encode(&map_k, a.kcache, 4, dims, strides, box);
    if (rc) return rc;
    rc = encode(&map_v, a.vcache, 4, dims, strides, box);
    if (rc) return rc;
  }
  AtcArgs args;
  args.a = a;
  args.num_pages = num_pages;
  args.status = status;
  const size_t tile_bytes = (size_t)(a.d / 64) * ATC_HALF_BYTES;
  const size_t smem = 5 * tile_bytes + ATC_P_BYTES + 1024;     // Q, 2 K, 2 V, P
  cudaError_t e;
  if (a.d == 128) {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc: %s", cudaGetErrorString(e));
      set = true;
    }
    e = gg_launch(attn_prefill_tc_kernel<128>, dim3(a.nh, num_tiles), dim3(ATC_THREADS), smem, stream, map_q, map_k,
                  map_v, args);
  } else {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc: %s", cudaGetErrorString(e));
      set = true;
    }
    e = gg_launch(attn_prefill_tc_kernel<64>, dim3(a.nh, num_tiles), dim3(ATC_THREADS), smem, stream, map_q, map_k,
                  map_v, args);
  }
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("attn_prefill_tc");
}
