// Causal attention of prompt portions on tcgen05, two heads of a kv head per CTA as in
// attention_tc2.cu, but in steps of 128 keys, with a row's 128 scores in the registers of one
// thread: half as many products to issue and half as many hand-overs between the roles per
// key as with 64.  bfloat16, head sizes 64 and 128, pages of up to 128 tokens.
//
// Same contract as the other prompt kernels (attention.cu, attention_mma.cu, attention_tc.cu,
// attention_tc2.cu): keys and values come only from the paged cache through the sequence's
// block table, masking is by absolute position (and an optional window), kv head = head /
// (nh/nkv), scale 1/sqrt(d).
//
// Twelve warps in three groups of four:
//   warp 0      TMA: both Q tiles once, then per step the K and V tiles of 128 keys (lane p
//               fetches page p; a page that is not there is asked for past the end and comes
//               back as zeros).  Two stages each for K and V.
//   warps 1, 2  one lane of each issues the MMAs of one head: S_h = Q_h K^T (128 x 128 x d) into
//               the head's score buffer in tensor memory, then O_h += P_h V (V as an MN-major
//               operand, P from tensor memory) when the head's P has arrived, then the next
//               scores over the P just used: the tensor core runs one thread's instructions in
//               the order they were issued.  While a head's softmax threads work, the tensor
//               core multiplies for the other head.  (warp 3 has nothing to do.)
//   warps 4-7   softmax of head 0, warps 8-11 of head 1: one thread per query row (row = tensor
//               memory lane), the row's 128 scores read once with tcgen05.ld, base-2
//               exponentials against a reference maximum that only moves (and O is only
//               rescaled, through tcgen05.ld/st) when a row of the warp has outgrown it by 2^8;
//               P goes back into tensor memory as pairs of bfloat16 over the first 64 columns
//               of the scores it came from.
// 128 scores and their exponentials need more registers than a third of the register file
// divided by 384 threads: the first group of warps gives registers back (setmaxnreg.dec) and
// the softmax groups take them (setmaxnreg.inc).  The launcher checks that what the kernel
// was given at launch covers both numbers, since a group that asks for more than there is
// waits for ever.
// Tensor memory per head: columns [0, 128) scores / P, [128, 128 + d) O; head 1 at +256.
// All waits on barriers are bounded; a wait that runs out sets *status and the CTA winds down.
#include "attention_common.cuh"
#include "tc_common.cuh"

#define AT3_BQ 128
#define AT3_BK 128
#define AT3_THREADS 384
#define AT3_HALF (128 * 128)                 // [128 rows x 64 columns] bf16, rows of 128 bytes, swizzled
#define AT3_LOG2E 1.4426950408889634f
#define AT3_REGS_FEW 56                      // registers a thread of warps 0-3 keeps
#define AT3_REGS_MANY 224                    // registers a softmax thread takes
#define AT3_POOL (128 * AT3_REGS_FEW + 256 * AT3_REGS_MANY)

enum { AT3_ERR_PRODUCER = 61, AT3_ERR_MMA = 62, AT3_ERR_SOFTMAX = 63 };

__device__ __forceinline__ void at3_mma(unsigned d_tmem, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi,
                                        unsigned idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"((unsigned)accumulate), "r"(0u)
      : "memory");
}
// The same with the A operand in tensor memory (lanes = rows, a 32-bit column = two bfloat16 of k).
__device__ __forceinline__ void at3_mma_ta(unsigned d_tmem, unsigned a_tmem, unsigned b_lo, unsigned b_hi,
                                           unsigned idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, {%6, %6, %6, %6}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"((unsigned)accumulate), "r"(0u)
      : "memory");
}

// Arithmetic of sm_100 that halves the softmax's instruction count: the maximum of three, and
// two float32 operations in one instruction on a pair of registers.
__device__ __forceinline__ float at3_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (x0, x1) * m + c
__device__ __forceinline__ void at3_fma2(float& r0, float& r1, float x0, float x1, float m, float c) {
  asm("{\n\t.reg .b64 pa, pb, pc, pd;\n\t"
      "mov.b64 pa, {%2, %3};\n\tmov.b64 pb, {%4, %4};\n\tmov.b64 pc, {%5, %5};\n\t"
      "fma.rn.f32x2 pd, pa, pb, pc;\n\tmov.b64 {%0, %1}, pd;\n\t}"
      : "=f"(r0), "=f"(r1) : "f"(x0), "f"(x1), "f"(m), "f"(c));
}
// (a0, a1) += (x0, x1)
__device__ __forceinline__ void at3_add2(float& a0, float& a1, float x0, float x1) {
  asm("{\n\t.reg .b64 pa, pb, pd;\n\t"
      "mov.b64 pa, {%0, %1};\n\tmov.b64 pb, {%2, %3};\n\t"
      "add.rn.f32x2 pd, pa, pb;\n\tmov.b64 {%0, %1}, pd;\n\t}"
      : "+f"(a0), "+f"(a1) : "f"(x0), "f"(x1));
}

struct At3Args {
  AttnArgs a;
  int num_pages;          // pages in the cache (an index >= this is filled with zeros)
  int* status;
};

template <int D>
__global__ void __launch_bounds__(AT3_THREADS, 1)
attn_prefill_tc3_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const At3Args args) {
  extern __shared__ unsigned char at3_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[20];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  constexpr int HALVES = D / 64;
  constexpr unsigned TILE_BYTES = HALVES * AT3_HALF;      // a Q, K or V tile: 128 rows x D
  const AttnArgs& a = args.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned base = (tc_smem(at3_smem_raw) + 1023u) & ~1023u;
  const unsigned q_smem = base;                                   // [2 heads]
  const unsigned k_smem = q_smem + 2 * TILE_BYTES;                // [2 stages]
  const unsigned v_smem = k_smem + 2 * TILE_BYTES;                // [2 stages]
  // barriers: 0 q_full; 1,2 k_full; 3,4 k_empty; 5,6 v_full; 7,8 v_empty;
  // per head t (base 9 + 4 t): +0 s_full, +1 p_full, +2 pv_done, +3 turn
  const unsigned q_full = tc_smem(&bars[0]), k_full0 = tc_smem(&bars[1]), k_empty0 = tc_smem(&bars[3]),
                 v_full0 = tc_smem(&bars[5]), v_empty0 = tc_smem(&bars[7]);
  auto s_full = [&](int t) { return tc_smem(&bars[9 + 4 * t]); };
  auto p_full = [&](int t) { return tc_smem(&bars[9 + 4 * t + 1]); };
  auto pv_done = [&](int t) { return tc_smem(&bars[9 + 4 * t + 2]); };
  auto turn = [&](int t) { return tc_smem(&bars[9 + 4 * t + 3]); };     // head t may run its exponentials

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 2);
      mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 2);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 4);
      mbar_init(pv_done(t), 1);
      mbar_init(turn(t), 4);
    }
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

  // ---- what this CTA works on: grid (head pairs, tiles), the tiles with the most keys first
  // (the lists were copied in before the step began: read before the wait)
  const int b = a.tile_seq[blockIdx.y], q0 = a.tile_q0[blockIdx.y];
  const int h0 = 2 * blockIdx.x, kvh = h0 / (a.nh / a.nkv);
  const int t0 = a.cu_q_lens[b], qlen = a.cu_q_lens[b + 1] - t0;
  const int ctx = a.context_lens[b];
  const int qstart = ctx - qlen;
  const int nrows = min(AT3_BQ, qlen - q0);
  const int first = qstart + q0;                       // position of the tile's first query
  const int hi = first + nrows;
  const int lo = a.window > 0 ? max(0, first - a.window + 1) : 0;
  const int kstart = (lo / AT3_BK) * AT3_BK;
  const int ntiles = (hi - kstart + AT3_BK - 1) / AT3_BK;
  const int ps = a.page_size, pages_per_tile = AT3_BK / ps;
  pdl_wait();

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(AT3_REGS_FEW));
    if (warp == 0) {
      // ---------------- TMA producer
      const int* bt = a.block_tables + (size_t)b * a.bt_stride;
      if (lane == 0) {
        mbar_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf)
            tma_load_2d(q_smem + t * TILE_BYTES + hf * AT3_HALF, &map_q, (h0 + t) * D + hf * 64, t0 + q0, q_full);
      }
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        const unsigned phase = (j >> 1) & 1;
        const int kb = kstart + j * AT3_BK;
        int page = -1;
        if (lane < pages_per_tile) {
          const int tok = kb + lane * ps;
          if (tok < hi && tok + ps > lo) page = __ldg(bt + tok / ps);
          if (page < 0) page = args.num_pages;                   // past the end: TMA fills zeros
        }
        const unsigned row_off = (unsigned)(lane * ps * 128);
        for (int which = 0; which < 2 && ok; ++which) {          // keys, then values
          const unsigned full = (which ? v_full0 : k_full0) + 8 * s, empty = (which ? v_empty0 : k_empty0) + 8 * s;
          const unsigned dst = (which ? v_smem : k_smem) + s * TILE_BYTES;
          const CUtensorMap* map = which ? &map_v : &map_k;
          ok = mbar_wait(empty, phase ^ 1) && !*(volatile int*)&abort_s;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (lane == 0) mbar_expect_tx(full, TILE_BYTES);
          __syncwarp();
          if (lane < pages_per_tile) {
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf)
              tma_load_4d(dst + hf * AT3_HALF + row_off, map, hf * 64, 0, kvh, page, full);
          }
        }
      }
      if (!ok && lane == 0) { atomicExch(args.status, AT3_ERR_PRODUCER); atomicExch(&abort_s, 1); }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ---------------- MMA issuers: one lane of warp 1 for head 0, one of warp 2 for head 1.
      // A key or value tile is free when both have committed (those barriers count two arrivals).
      const int t = warp - 1;
      // instruction descriptors: f32 accumulate, bf16 inputs, M = 128; scores: N = 128 keys
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
      // O += P V: N = D, B (V) is MN-major
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (((unsigned)D >> 3) << 17) | ((128u >> 4) << 24);
      // the descriptors' upper words never change and a tile's k step only adds to the address
      // field of the lower word
      const unsigned hi_k = 64u | (1u << 14) | (2u << 29);                 // SBO 1024 bytes, version 1, 128-byte swizzle
      const unsigned lbo_k = 1u << 16, lbo_v = (unsigned)(AT3_HALF >> 4) << 16;
      auto lo_word = [](unsigned addr, unsigned lbo) { return ((addr & 0x3FFFFu) >> 4) | lbo; };
      const unsigned q_lo = lo_word(q_smem + t * TILE_BYTES, lbo_k);
      unsigned k_lo[2], v_lo[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        k_lo[i] = lo_word(k_smem + i * TILE_BYTES, lbo_k);
        v_lo[i] = lo_word(v_smem + i * TILE_BYTES, lbo_v);
      }
      const unsigned tmem_s = tmem_base + t * 256, tmem_o = tmem_s + 128;
      bool ok = mbar_wait(q_full, 0);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(k_full0 + 8 * s, (j >> 1) & 1)) return false;
        // the score buffer is free: the product that read P from it was issued before this
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const unsigned off = ((k >> 2) * AT3_HALF + (k & 3) * 32) >> 4;
          at3_mma(tmem_s, q_lo + off, hi_k, k_lo[s] + off, hi_k, idesc_qk, k > 0);
        }
        tc_commit(s_full(t));                // this head's scores ready
        tc_commit(k_empty0 + 8 * s);         // this head is done with the key tile
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (*(volatile int*)&abort_s) { ok = false; break; }
        const int s = j & 1;
        if (!mbar_wait(v_full0 + 8 * s, (j >> 1) & 1)) { ok = false; break; }
        if (!mbar_wait(p_full(t), j & 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT3_BK / 16; ++k) {
          // A = P from tensor memory: 16 keys = 8 columns.  B = V (MN-major: d contiguous): 16
          // keys further = 16 rows of 128 bytes; the second half of d is one half tile (LBO)
          // further; groups of 8 keys are 1024 bytes apart (SBO)
          at3_mma_ta(tmem_o, tmem_s + k * 8, v_lo[s] + ((k * 16 * 128) >> 4), hi_k, idesc_pv, j > 0 || k > 0);
        }
        tc_commit(pv_done(t));               // O of this head holds the step
        tc_commit(v_empty0 + 8 * s);         // this head is done with the value tile
        if (j + 1 < ntiles) ok = issue_qk(j + 1);
      }
      if (!ok) { atomicExch(args.status, AT3_ERR_MMA); atomicExch(&abort_s, 1); }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(AT3_REGS_MANY));
    // ---------------- softmax and epilogue: warps 4-7 head h0, warps 8-11 head h0 + 1; a warp reads
    // the tensor-memory lanes of its quarter (warp % 4); one thread per query row
    const int t = (warp - 4) >> 2, quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int pos = first + r;
    const bool row_ok = r < nrows;
    const unsigned lane_addr = tmem_base + t * 256 + ((unsigned)(quarter * 32) << 16);
    const unsigned tmem_o = lane_addr + 128;
    const float sc = a.scale * AT3_LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    const int stale_hi = (hi + ps - 1) / ps * ps;        // end of the last page that is fetched
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
      const int kb = kstart + j * AT3_BK;
      ok = mbar_wait(s_full(t), j & 1) && !*(volatile int*)&abort_s;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool interior = kb >= lo && kb + AT3_BK - 1 <= first && (a.window <= 0 || kb > first + nrows - 1 - a.window);
      // the row's 128 scores, once, into registers (as they come: the scale to base 2 is folded
      // into the exponential's argument; masked ones -inf).  The four loads are in flight together.
      float sv[AT3_BK];
      {
        unsigned raw[AT3_BK];
#pragma unroll
        for (int c = 0; c < AT3_BK; c += 32) tc_load32_nowait(lane_addr + c, raw + c);
        tc_wait_load();
#pragma unroll
        for (int i = 0; i < AT3_BK; ++i) sv[i] = __uint_as_float(raw[i]);
      }
      if (!interior) {
#pragma unroll
        for (int i = 0; i < AT3_BK; ++i) {
          const int tk = kb + i;
          const bool keep = row_ok && tk >= lo && tk <= pos && (a.window <= 0 || tk > pos - a.window);
          if (!keep) sv[i] = -INFINITY;
        }
      }
      // the maximum, three at a time in four chains (a chain of 128 dependent operations would be
      // 128 latencies long, and there is one softmax warp per scheduler at work at a time)
      float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < AT3_BK; i += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mxs[u] = at3_max3(mxs[u], sv[i + 2 * u], sv[i + 2 * u + 1]);
      }
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * sc;      // sc > 0
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
      if (j > 0 && rescale) {
        // The product of the step before is complete: these scores were multiplied after it by
        // the same thread, and the commit behind them (s_full) covers everything it had issued.
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          unsigned v[32];
          tc_load32(tmem_o + c, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tc_store32(tmem_o + c, v);
        }
        tc_wait_store();
      }
      // The last page of the last tile may hold rows past the context: whatever the page's
      // owner before left there.  Their P is zero, but zero times a NaN or an infinity is not:
      // those rows of V are cleared before the product reads them (by each head's own warps,
      // whose arrival on p_full the product waits for).
      if (j == ntiles - 1 && stale_hi > ctx) {
        ok = mbar_wait(v_full0 + 8 * s, (j >> 1) & 1) && !*(volatile int*)&abort_s;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int z0 = max(ctx, kb) - kb, z1 = min(stale_hi, kb + AT3_BK) - kb;
        if (r >= z0 && r < z1) {
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf) {
            const unsigned row = v_smem + s * TILE_BYTES + hf * AT3_HALF + (unsigned)r * 128;
#pragma unroll
            for (int c = 0; c < 128; c += 16)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(row + c), "r"(0u) : "memory");
          }
        }
        fence_async_smem();
      }
      // The exponentials of the two heads take turns (head 0 first in every step): the special
      // function unit serves one head at full rate while the other head's warps wait for the
      // tensor core or read tensor memory, instead of both queueing for each in step.
      ok = mbar_wait(turn(t), t == 0 ? ((j & 1) ^ 1) : (j & 1)) && !*(volatile int*)&abort_s;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // p = 2^(s * scale - m_ref), row sum, P into the first 64 columns of the score buffer
      // (column c = keys 2c, 2c + 1 as a pair of bfloat16); the argument and the sum two at a time
      const float neg_mr = m_ref == -INFINITY ? 0.f : -m_ref;
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < AT3_BK; c += 64) {
        unsigned pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float a0, a1;
          at3_fma2(a0, a1, sv[c + i], sv[c + i + 1], sc, neg_mr);           // -inf stays -inf
          const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);               // 2^-inf = 0
          at3_add2(sums[i & 2], sums[(i & 2) + 1], p0, p1);
          __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
          pk[i >> 1] = *reinterpret_cast<unsigned*>(&pr);
        }
        tc_store32(lane_addr + (c >> 1), pk);
      }
      l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
      tc_wait_store();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(p_full(t)); mbar_arrive(turn(1 - t)); }
    }
    if (ok && ntiles > 0) {
      ok = mbar_wait(pv_done(t), (ntiles - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0) { atomicExch(args.status, AT3_ERR_SOFTMAX); atomicExch(&abort_s, 1); }
    tc_fence_after();
    if (ok && !*(volatile int*)&abort_s) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)(t0 + q0 + r) * a.nh * D + (size_t)(h0 + t) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
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
// Registers the kernel is given at launch, times its threads: what the two setmaxnreg numbers
// must fit into.  0 if the kernel cannot be asked.
template <int D> static int at3_register_pool() {
  static int pool = -1;
  if (pool < 0) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, attn_prefill_tc3_kernel<D>) != cudaSuccess) { (void)cudaGetLastError(); pool = 0; }
    else pool = fa.numRegs * AT3_THREADS;
  }
  return pool;
}

bool attn_tc3_supported(int dtype, int d, int page_size, int nh, int nkv) {
  if (!(dtype == GG_BF16 && (d == 64 || d == 128) && page_size >= 8 && page_size <= AT3_BK &&
        (page_size & (page_size - 1)) == 0 && nkv > 0 && nh % nkv == 0 && (nh / nkv) % 2 == 0))
    return false;
  // a softmax group that asks for more registers than the CTA was given would wait for ever
  return (d == 128 ? at3_register_pool<128>() : at3_register_pool<64>()) >= AT3_POOL;
}

static int encode3(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box) {
  GgEncodeTiledFn fn = gg_encode_tiled();
  if (!fn) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc3: the driver has no cuTensorMapEncodeTiled");
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc3: cuTensorMapEncodeTiled failed with %d", (int)r);
  return GG_OK;
}

// a.tile_seq / a.tile_q0 list tiles of 128 query rows.  T = rows of the q buffer.
int attn_prefill_tc3(const AttnArgs& a, int num_tiles, int T, int num_pages, int* status, cudaStream_t stream) {
  GG_REQUIRE(num_tiles >= 0 && num_tiles <= 65535, "attn_prefill_tc3: %d tiles in one launch", num_tiles);
  GG_REQUIRE(status != nullptr, "attn_prefill_tc3: no status word given");
  GG_REQUIRE(a.q_stride % 8 == 0 && ((size_t)a.q % 16) == 0, "attn_prefill_tc3: q rows must be 16-byte aligned");
  GG_REQUIRE((a.nh / a.nkv) % 2 == 0, "attn_prefill_tc3: %d heads per kv head; pairs of heads must share a kv head", a.nh / a.nkv);
  GG_REQUIRE(attn_tc3_supported(GG_BF16, a.d, a.page_size, a.nh, a.nkv), "attn_prefill_tc3: not for this shape or build");
  if (num_tiles == 0) return GG_OK;
  CUtensorMap map_q, map_k, map_v;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a.nh * a.d, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)a.q_stride * 2};
    cuuint32_t box[2] = {64, AT3_BQ};
    int rc = encode3(&map_q, a.q, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t D = (cuuint64_t)a.d;
    cuuint64_t dims[4] = {D, (cuuint64_t)a.page_size, (cuuint64_t)a.nkv, (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {D * 2, (cuuint64_t)a.page_size * D * 2, (cuuint64_t)a.nkv * a.page_size * D * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)a.page_size, 1, 1};
    int rc = encode3(&map_k, a.kcache, 4, dims, strides, box);
    if (rc) return rc;
    rc = encode3(&map_v, a.vcache, 4, dims, strides, box);
    if (rc) return rc;
  }
  At3Args args;
  args.a = a;
  args.num_pages = num_pages;
  args.status = status;
  const size_t halves = (size_t)(a.d / 64);
  const size_t smem = 6 * halves * AT3_HALF + 1024;   // 2 Q, 2 K, 2 V
  cudaError_t e;
  if (a.d == 128) {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attn_prefill_tc3_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc3: %s", cudaGetErrorString(e));
      set = true;
    }
    e = gg_launch(attn_prefill_tc3_kernel<128>, dim3(a.nh / 2, num_tiles), dim3(AT3_THREADS), smem, stream, map_q,
                  map_k, map_v, args);
  } else {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attn_prefill_tc3_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc3: %s", cudaGetErrorString(e));
      set = true;
    }
    e = gg_launch(attn_prefill_tc3_kernel<64>, dim3(a.nh / 2, num_tiles), dim3(AT3_THREADS), smem, stream, map_q,
                  map_k, map_v, args);
  }
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_prefill_tc3: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("attn_prefill_tc3");
}
