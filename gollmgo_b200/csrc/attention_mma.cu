// Attention over the paged cache on the tensor cores, bfloat16, head sizes 64 and 128.
//
// Same contract as the general kernels in attention.cu (same formulas: kv head =
// head / (nh/nkv), scale 1/sqrt(d), causal by absolute position, optional window,
// keys only from the cache through the block table), different machinery:
//   * keys and values of 64 tokens at a time are brought to shared memory with
//     16-byte cp.async copies (zero-filled past the end or where a page was given
//     back), three stages deep for decode and two for prompts, in a layout whose
//     16-byte columns are XOR-swizzled by the row so ldmatrix has no bank conflicts;
//   * scores S = Q K^T and outputs O += P V are mma.sync m16n8k16 (bf16 in, f32
//     accumulate); P goes from the score accumulators straight into the A operand;
//   * softmax is online in float32 with base-2 exponentials (scores are scaled by
//     scale * log2(e)).
// Decode: one CTA per (token, kv head [x 16 heads of its group], slice of the
// context); the 16 rows of the A operand are the query heads that share the kv
// head, so every key and value is read once per group; the four warps take 16
// keys each of every 64 and are combined through shared memory at the end.
// Prompt portions: one CTA per (64 queries of a sequence, head); a warp owns 16
// query rows.
#include "attention_common.cuh"
#include <cstdlib>

#define MMA_THREADS 128
#define MMA_BK 64
#define DEC_BT_CACHE 512          // block-table entries a decode CTA keeps in shared memory
#define LOG2E 1.4426950408889634f

bool attn_mma_supported(int dtype, int d) { return dtype == GG_BF16 && (d == 64 || d == 128); }
static bool power_of_two(int x) { return x > 0 && (x & (x - 1)) == 0; }

// Shared-memory tile [64 rows][D] bf16; the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
template <int D> __device__ __forceinline__ unsigned tile_off(int row, int chunk) {
  return (unsigned)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Bring keys and values of tokens [k0, k0+64) of one sequence and kv head to a stage.
// Tokens outside [lo, hi) and pages that were given back are zero-filled.  The page size
// is a power of two (ps_log2), so the page of a token is a shift away.
// bt_local: bt points to a copy of the block table in shared memory (plain loads).
template <int D, bool BT_LOCAL = false>
__device__ __forceinline__ void load_kv_tile(const AttnArgs& a, const int* bt, int kvh, int k0, int lo,
                                             int hi, unsigned ks, unsigned vs, int ps_log2) {
  constexpr int CPR = D / 8;                       // 16-byte chunks per row
  constexpr int ROWS_PER_PASS = MMA_THREADS / CPR;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)a.kcache;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)a.vcache;
  const int ch = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
  const int ps_mask = (1 << ps_log2) - 1;
  const size_t page_elems = (size_t)a.nkv << ps_log2;          // rows of D elements per page
  const unsigned in_head = ((unsigned)kvh << ps_log2);
#pragma unroll
  for (int i = 0; i < MMA_BK / ROWS_PER_PASS; ++i) {
    const int row = r0 + i * ROWS_PER_PASS;
    const int tok = k0 + row;
    int page = -1;
    if (tok >= lo && tok < hi) page = BT_LOCAL ? bt[tok >> ps_log2] : __ldg(bt + (tok >> ps_log2));
    const size_t src = page >= 0 ? ((size_t)page * page_elems + in_head + (unsigned)(tok & ps_mask)) * D + ch * 8 : 0;
    const int bytes = page >= 0 ? 16 : 0;
    const unsigned off = tile_off<D>(row, ch);
    cp_async16(ks + off, kc + src, bytes);
    cp_async16(vs + off, vc + src, bytes);
  }
}

// Scores of 16 query rows against NT*8 keys (rows key0.. of the staged tile).
template <int D, int NT>
__device__ __forceinline__ void qk_mma(const unsigned (*qf)[4], unsigned ks, int key0, float (*s)[4]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      // four 8x8 matrices: (keys j*8.., d chunk 2kk), (same keys, chunk 2kk+1), (keys (j+1)*8.., 2kk), (.., 2kk+1)
      const int mi = lane >> 3;
      const int row = key0 + (j + (mi >> 1)) * 8 + (lane & 7);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, ks + tile_off<D>(row, 2 * kk + (mi & 1)));
      mma_bf16(s[j], qf[kk], b0, b1);
      mma_bf16(s[j + 1], qf[kk], b2, b3);
    }
  }
}

// O(16 x D) += P(16 x NT*8) V(NT*8 x D); p holds NT/2 A-operand fragments.
template <int D, int NT>
__device__ __forceinline__ void pv_mma(const unsigned (*p)[4], unsigned vs, int key0, float (*o)[4]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
    for (int nt = 0; nt < D / 8; nt += 2) {
      // (keys kk*16.. +8, d chunk nt), (keys +8.. +16, chunk nt), (keys ..+8, chunk nt+1), (keys +8.., chunk nt+1)
      const int mi = lane >> 3;
      const int row = key0 + kk * 16 + (mi & 1) * 8 + (lane & 7);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vs + tile_off<D>(row, nt + (mi >> 1)));
      mma_bf16(o[nt], p[kk], b0, b1);
      mma_bf16(o[nt + 1], p[kk], b2, b3);
    }
  }
}

// One online-softmax update of a warp's 16 rows with NT*8 new scores (already scaled
// to base 2 and masked with -inf).  Thread holds rows g = lane/4 (regs 0,1) and g+8 (2,3).
template <int D, int NT>
__device__ __forceinline__ void softmax_update(float (*s)[4], float* m, float* l, float (*o)[4],
                                               unsigned (*p)[4]) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
  const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
  const float al0 = fast_exp2(m[0] - ref0), al1 = fast_exp2(m[1] - ref1);
  m[0] = mn0;
  m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    s[j][0] = fast_exp2(s[j][0] - ref0);
    s[j][1] = fast_exp2(s[j][1] - ref0);
    s[j][2] = fast_exp2(s[j][2] - ref1);
    s[j][3] = fast_exp2(s[j][3] - ref1);
    sum0 += s[j][0] + s[j][1];
    sum1 += s[j][2] + s[j][3];
  }
  l[0] = l[0] * al0 + sum0;          // per-thread partial sums; the quad is reduced at the end
  l[1] = l[1] * al1 + sum1;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    o[nt][0] *= al0; o[nt][1] *= al0; o[nt][2] *= al1; o[nt][3] *= al1;
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    p[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    p[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    p[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    p[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
  }
}

// A-operand fragments of 16 query rows: row r of the tile is at qrow(r) (null = zero row).
template <int D, typename F>
__device__ __forceinline__ void load_q_frags(unsigned (*qf)[4], F qrow) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = (lane & 3) * 2;
  const __nv_bfloat16* r0 = qrow(g);
  const __nv_bfloat16* r1 = qrow(g + 8);
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    qf[kk][0] = r0 ? *reinterpret_cast<const unsigned*>(r0 + kk * 16 + c) : 0u;
    qf[kk][1] = r1 ? *reinterpret_cast<const unsigned*>(r1 + kk * 16 + c) : 0u;
    qf[kk][2] = r0 ? *reinterpret_cast<const unsigned*>(r0 + kk * 16 + c + 8) : 0u;
    qf[kk][3] = r1 ? *reinterpret_cast<const unsigned*>(r1 + kk * 16 + c + 8) : 0u;
  }
}

// ---------------------------------------------------------------- decoded tokens
// CLUSTER: the slices of one (token, kv head) are the CTAs of a thread-block cluster
// (1, 1, slices) and merge their results through distributed shared memory, every CTA
// writing its share of the output; otherwise a CTA leaves its slice's result in part_o /
// part_ml for the merge kernel.
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }
// v into the same shared-memory address of CTA `rank` of the cluster
__device__ __forceinline__ void st_cluster_f32(unsigned local_addr, unsigned rank, float v) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "st.shared::cluster.f32 [ra], %2;\n\t}"
      :: "r"(local_addr), "r"(rank), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(unsigned local_addr, unsigned rank) {
  float v;
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %1, %2;\n\t"
      "ld.shared::cluster.f32 %0, [ra];\n\t}"
      : "=f"(v) : "r"(local_addr), "r"(rank) : "memory");
  return v;
}

// ROPE: what rope_kv_write does for a decoded token (rope_cache.cu, the same arithmetic),
// inside this kernel: cosines and sines of the token's position into `scratch`, the CTA's
// query heads rotated into scratch (bfloat16, [16][D]), and, in the one CTA whose slice holds
// the token's own position, k rotated and v copied into their place in the cache.  Half-split
// pairs over the whole head.  Ends with a barrier: the CTA then sees q and the new k and v.
// The table of cosines and sines depends only on the token's position (known before the
// step began): decode_rope_table may run before the wait on the kernels ahead.
template <int D>
__device__ __forceinline__ void decode_rope_table(const AttnArgs& a, int t, unsigned char* scratch) {
  float* cs = reinterpret_cast<float*>(scratch);
  constexpr int half = D / 2;
  const double pos = (double)a.rope_positions[t];
  const double two_pi = 6.283185307179586476925286766559;
  for (int p = threadIdx.x; p < half; p += MMA_THREADS) {
    const double ang = pos * a.rope_inv_freq[p];
    const float r = (float)(ang - two_pi * rint(ang * (1.0 / two_pi)));
    float sn, c;
    sincosf(r, &sn, &c);
    cs[p] = c;
    cs[half + p] = sn;
  }
}

template <int D>
__device__ __forceinline__ void decode_rope(const AttnArgs& a, int t, int kvh, int head0, int nrows, bool owner,
                                            unsigned char* scratch) {
  float* cs = reinterpret_cast<float*>(scratch);
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(scratch + D * sizeof(float));
  constexpr int half = D / 2, per_head = half / 8;
  __syncthreads();                       // the table is complete
  const int slot = (owner && a.rope_write_cache && a.slot_mapping) ? a.slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / a.page_size : 0;
  const int off = slot >= 0 ? slot - page * a.page_size : 0;
  const __nv_bfloat16* row = (const __nv_bfloat16*)a.q + (size_t)t * a.q_stride;
  const size_t cache_row = (((size_t)page * a.nkv + kvh) * a.page_size + off) * D;
  const int q_items = nrows * per_head, k_items = slot >= 0 ? per_head : 0, v_items = slot >= 0 ? D / 8 : 0;
  for (int e = threadIdx.x; e < q_items + k_items + v_items; e += MMA_THREADS) {
    if (e < q_items + k_items) {
      const bool is_k = e >= q_items;
      const int hh = is_k ? 0 : e / per_head;
      const int p0 = (is_k ? e - q_items : e - hh * per_head) << 3;
      const __nv_bfloat16* x = row + (size_t)(is_k ? a.nh + kvh : head0 + hh) * D;
      uint4 lo = *reinterpret_cast<const uint4*>(x + p0), hi = *reinterpret_cast<const uint4*>(x + half + p0);
      __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&lo);
      __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 av = __bfloat1622float2(a2[i]), bv = __bfloat1622float2(b2[i]);
        const float c0 = cs[p0 + 2 * i], s0 = cs[half + p0 + 2 * i], c1 = cs[p0 + 2 * i + 1], s1 = cs[half + p0 + 2 * i + 1];
        a2[i] = __floats2bfloat162_rn(av.x * c0 - bv.x * s0, av.y * c1 - bv.y * s1);
        b2[i] = __floats2bfloat162_rn(av.x * s0 + bv.x * c0, av.y * s1 + bv.y * c1);
      }
      __nv_bfloat16* dst = is_k ? (__nv_bfloat16*)a.kcache + cache_row : qs + hh * D;
      *reinterpret_cast<uint4*>(dst + p0) = lo;
      *reinterpret_cast<uint4*>(dst + half + p0) = hi;
    } else {
      const int c = (e - q_items - k_items) << 3;
      *reinterpret_cast<uint4*>((__nv_bfloat16*)a.vcache + cache_row + c) =
          *reinterpret_cast<const uint4*>(row + (size_t)(a.nh + a.nkv + kvh) * D + c);
    }
  }
  __syncthreads();
}

template <int D, int STAGES, bool CLUSTER, bool ROPE>
__global__ void __launch_bounds__(MMA_THREADS, D == 128 ? 3 : 4) attn_decode_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // The merge's inbox, behind the ring: every slice of the cluster leaves its share of the
  // result here (and its row maxima and sums with everybody), so a CTA merges from its own
  // shared memory.  A place of its own: neighbours write it while this CTA may still be in
  // its loop.  Sized for the rows there are (decode_inbox_bytes): what a CTA holds in shared
  // memory decides whether the next kernel's CTAs can settle beside it and fetch their
  // weights while this one finishes.
  float* rx_ml = reinterpret_cast<float*>(smem_raw + STAGES * 2 * MMA_BK * D * 2);   // [slices][16][2]
  float* rx_o = rx_ml + ATTN_MAX_CLUSTER * 32;                                     // [slices][per]
  // nobody may write a neighbour's shared memory before that neighbour runs: everybody
  // arrives here, and waits for the others only just before the first such write
  if (CLUSTER) cluster_arrive_relaxed();
  constexpr int TILE_BYTES = MMA_BK * D * 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c2 = (lane & 3) * 2;
  // The lists that say what this CTA works on were copied in before the step began, and
  // keys of earlier steps are in the cache already: only the newest key and the queries
  // come from the kernels just before this one.
  const int ps_log2 = 31 - __clz(a.page_size);
  const int G = a.nh / a.nkv, gchunks = (G + 15) / 16;
  const int b = a.dec_seqs[blockIdx.x];
  const int kvh = blockIdx.y / gchunks, g0 = (blockIdx.y % gchunks) * 16;
  const int split = blockIdx.z, S = a.num_splits;
  const int nrows = min(16, G - g0);
  const int ctx = b >= 0 ? a.context_lens[b] : 0;
  const int t = b >= 0 ? a.cu_q_lens[b] : 0;
  const int lo0 = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int n = ctx - lo0;
  int chunk = (n + S - 1) / S;
  chunk = ((chunk + MMA_BK - 1) / MMA_BK) * MMA_BK;
  const int lo = lo0 + split * chunk, hi = min(ctx, lo + chunk);
  const int head0 = kvh * G + g0;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }

  // the first tiles can be fetched before the kernels ahead have finished, unless they
  // hold the key this step wrote (position ctx - 1)
  // the slice's part of the block table, once, into shared memory: a tile's copies then start
  // without a look-up in global memory first
  __shared__ int bt_s[DEC_BT_CACHE];
  const int pg_first = lo >> ps_log2, n_pg = lo < hi ? ((hi - 1) >> ps_log2) - pg_first + 1 : 0;
  const bool bt_local = n_pg > 0 && n_pg <= DEC_BT_CACHE;
  if (bt_local) {
    const int* btg = a.block_tables + (size_t)b * a.bt_stride + pg_first;
    for (int i = threadIdx.x; i < n_pg; i += MMA_THREADS) bt_s[i] = __ldg(btg + i);
    __syncthreads();
  }
  // ROPE: the last stage is free until the main loop starts filling it
  unsigned char* scratch = smem_raw + (STAGES - 1) * 2 * TILE_BYTES;
  const bool owner = lo <= ctx - 1 && ctx - 1 < hi;
  if (ROPE && lo < hi) decode_rope_table<D>(a, t, scratch);
  const int* bt = bt_local ? bt_s - pg_first : a.block_tables + (size_t)b * a.bt_stride;
  const unsigned base = smem_u32(smem_raw);
  const int ntiles = lo < hi ? (hi - lo + MMA_BK - 1) / MMA_BK : 0;
  auto load_tile = [&](int i, int st) {
    if (bt_local) load_kv_tile<D, true>(a, bt, kvh, lo + i * MMA_BK, lo, hi, base + st * 2 * TILE_BYTES, base + st * 2 * TILE_BYTES + TILE_BYTES, ps_log2);
    else load_kv_tile<D, false>(a, bt, kvh, lo + i * MMA_BK, lo, hi, base + st * 2 * TILE_BYTES, base + st * 2 * TILE_BYTES + TILE_BYTES, ps_log2);
  };
  // the tiles that end before the key this step wrote (position ctx - 1) can be fetched
  // before the kernels ahead have finished: as many of them as the ring holds
  const int pre = lo < hi ? min(STAGES - 1, (ctx - 1 - lo) / MMA_BK) : 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < pre) { load_tile(s, s); cp_async_commit(); }
  }
  pdl_wait();
  if (ROPE && lo < hi) decode_rope<D>(a, t, kvh, head0, nrows, owner, scratch);
  if (lo < hi) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s >= pre) {
        if (s < ntiles) load_tile(s, s);
        cp_async_commit();
      }
    }
    unsigned qf[D / 16][4];
    const __nv_bfloat16* qbase = ROPE ? reinterpret_cast<const __nv_bfloat16*>(scratch + D * sizeof(float))
                                      : (const __nv_bfloat16*)a.q + (size_t)t * a.q_stride + (size_t)head0 * D;
    load_q_frags<D>(qf, [&](int r) { return r < nrows ? qbase + (size_t)r * D : nullptr; });
    if (ROPE) __syncthreads();           // the loop's first copy lands where q was
    const float sc = a.scale * LOG2E;
    for (int it = 0; it < ntiles; ++it) {
      const int nx = it + STAGES - 1;
      if (nx < ntiles) load_tile(nx, nx % STAGES);
      cp_async_commit();
      cp_async_wait<STAGES - 1>();
      __syncthreads();
      const int st = it % STAGES;
      const unsigned ks = base + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
      const int key0 = warp * 16;                        // this warp's 16 keys of the tile
      const int tok0 = lo + it * MMA_BK + key0;
      if (tok0 < hi) {
        float s[2][4];
        qk_mma<D, 2>(qf, ks, key0, s);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int tk = tok0 + j * 8 + c2;
          s[j][0] = tk < hi ? s[j][0] * sc : -INFINITY;
          s[j][2] = tk < hi ? s[j][2] * sc : -INFINITY;
          s[j][1] = tk + 1 < hi ? s[j][1] * sc : -INFINITY;
          s[j][3] = tk + 1 < hi ? s[j][3] * sc : -INFINITY;
        }
        unsigned p[1][4];
        softmax_update<D, 2>(s, m, l, o, p);
        pv_mma<D, 2>(p, vs, key0, o);
      }
      __syncthreads();
    }
    cp_async_wait<0>();
  }
  pdl_trigger();
  // ---- combine the four warps: (m, l, o) of each through shared memory
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  float* cm = reinterpret_cast<float*>(smem_raw);          // [4][16]
  float* cl = cm + 64;                                     // [4][16]
  float* co = cl + 64;                                     // [4][16][D]
  __syncthreads();
  if ((lane & 3) == 0) {
    cm[warp * 16 + g] = m[0]; cm[warp * 16 + g + 8] = m[1];
    cl[warp * 16 + g] = l[0]; cl[warp * 16 + g + 8] = l[1];
  }
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    float* r0 = co + ((size_t)warp * 16 + g) * D + nt * 8 + c2;
    float* r1 = co + ((size_t)warp * 16 + g + 8) * D + nt * 8 + c2;
    r0[0] = o[nt][0]; r0[1] = o[nt][1];
    r1[0] = o[nt][2]; r1[1] = o[nt][3];
  }
  __syncthreads();
  // CLUSTER: CTA s of the cluster merges elements [s * per, (s + 1) * per) of the rows; a
  // slice sends each of its elements to the CTA that merges it
  const int elems = nrows * D, per = ((elems / 2 + S - 1) / S) * 2;
  const unsigned rx_o_a = smem_u32(rx_o), rx_ml_a = smem_u32(rx_ml);
  if (CLUSTER) cluster_wait();
  for (int e = threadIdx.x; e < elems; e += MMA_THREADS) {
    const int r = e / D, col = e - r * D;
    float M = fmaxf(fmaxf(cm[r], cm[16 + r]), fmaxf(cm[32 + r], cm[48 + r]));
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = cm[w * 16 + r];
      if (mw != -INFINITY) {
        const float f = fast_exp2(mw - M);
        L += f * cl[w * 16 + r];
        acc += f * co[((size_t)w * 16 + r) * D + col];
      }
    }
    if (CLUSTER) {
      const int dest = e / per;
      st_cluster_f32(rx_o_a + (unsigned)(split * per + e - dest * per) * 4, dest, acc);
      if (col < S) {                     // threads col = 0 .. S-1 of the row: one neighbour each
        st_cluster_f32(rx_ml_a + (unsigned)(split * 32 + r * 2) * 4, col, M);
        st_cluster_f32(rx_ml_a + (unsigned)(split * 32 + r * 2 + 1) * 4, col, L);
      }
    } else {
      const size_t row = ((size_t)blockIdx.x * a.nh + head0 + r) * S + split;
      a.part_o[row * D + col] = acc;
      if (col == 0) {
        // the merge kernel works with natural exponentials: hand it m in that base
        a.part_ml[row * 2] = M == -INFINITY ? -INFINITY : M * (1.0f / LOG2E);
        a.part_ml[row * 2 + 1] = L;
      }
    }
  }
  if (CLUSTER) {
    // after this barrier every slice's numbers are in the inbox, and nobody touches a
    // neighbour's shared memory again: a CTA finishes on its own
    cluster_barrier();
    if (b >= 0) {
      __nv_bfloat16* out = (__nv_bfloat16*)a.out + (size_t)t * a.nh * D + (size_t)head0 * D;
      for (int i = 2 * threadIdx.x; i < per && split * per + i < elems; i += 2 * MMA_THREADS) {
        const int e = split * per + i, r = e / D, col = e - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < ATTN_MAX_CLUSTER; ++s)
          if (s < S) M = fmaxf(M, rx_ml[s * 32 + r * 2]);
        float L = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int s = 0; s < ATTN_MAX_CLUSTER; ++s) {
          if (s < S) {
            const float ms = rx_ml[s * 32 + r * 2];
            if (ms != -INFINITY) {
              const float f = fast_exp2(ms - M);
              const float2 v = *reinterpret_cast<const float2*>(rx_o + s * per + i);
              L += f * rx_ml[s * 32 + r * 2 + 1];
              o0 += f * v.x;
              o1 += f * v.y;
            }
          }
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        *reinterpret_cast<unsigned*>(out + (size_t)r * D + col) = pack_bf16(o0 * inv, o1 * inv);
      }
    }
  }
}

// ---------------------------------------------------------------- decoded tokens, large batches
// With more (token, kv head) pairs than CTAs fit at once, whole slices per CTA leave the
// last round of CTAs mostly empty.  Here the tiles of 64 keys of all pairs form one sequence
// (kv head chunk r outermost, then token, then tile), which is cut into gridDim.x equal
// ranges; a CTA walks its range with one ring of stages that runs on across the borders
// between pairs, and leaves one partial result (m, l, o of up to 16 heads) per pair it
// touched.  Piece number = (r * n_dec + token index) + CTA index: both only grow along the
// sequence, so the sum is unique, and attn_merge_flat_kernel finds a pair's pieces from the
// same arithmetic.  part_o [pieces, 16, D], part_ml [pieces, 16, 2] (m in base 2);
// prefix_out [n_dec + 1]: tiles before each token, written by CTA 0 for the merge kernel.
#define FLAT_MAX_SEQS 1024

struct FlatPos { int r, i, tt; };       // kv head chunk, decode entry, tile within the entry

template <int D>
__global__ void __launch_bounds__(MMA_THREADS, D == 128 ? 3 : 4)
attn_decode_flat_kernel(AttnArgs a, int n_dec, int* __restrict__ prefix_out) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int pre[FLAT_MAX_SEQS + 1];
  __shared__ float cm[64], cl[64];
  constexpr int TILE_BYTES = MMA_BK * D * 2;
  constexpr int STAGES = 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c2 = (lane & 3) * 2;
  const int ps_log2 = 31 - __clz(a.page_size);
  const int G = a.nh / a.nkv, gchunks = (G + 15) / 16, R = a.nkv * gchunks;

  // tiles of every entry (from the lists copied in before the step), then their prefix sums
  for (int i = threadIdx.x; i < n_dec; i += MMA_THREADS) {
    const int b = a.dec_seqs[i];
    const int ctx = b >= 0 ? a.context_lens[b] : 0;
    const int lo0 = a.window > 0 ? max(0, ctx - a.window) : 0;
    pre[i + 1] = (ctx - lo0 + MMA_BK - 1) / MMA_BK;
  }
  if (threadIdx.x == 0) pre[0] = 0;
  __syncthreads();
  if (warp == 0) {
    const int chunk = (n_dec + 31) / 32, s0 = lane * chunk, s1 = min(n_dec, s0 + chunk);
    int sum = 0;
    for (int i = s0; i < s1; ++i) sum += pre[i + 1];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = s0; i < s1; ++i) { run += pre[i + 1]; pre[i + 1] = run; }
  }
  __syncthreads();
  const int T_total = pre[n_dec];
  const long long U = (long long)R * T_total;
  const long long u_lo = (long long)blockIdx.x * U / gridDim.x, u_hi = (long long)(blockIdx.x + 1) * U / gridDim.x;
  const int ntiles = (int)(u_hi - u_lo);
  pdl_wait();
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i <= n_dec; i += MMA_THREADS) prefix_out[i] = pre[i];
  if (ntiles > 0) {
    auto advance = [&](FlatPos& p) {
      if (++p.tt == pre[p.i + 1] - pre[p.i]) {
        p.tt = 0;
        do {
          if (++p.i == n_dec) { p.i = 0; ++p.r; }
        } while (pre[p.i + 1] == pre[p.i] && p.r < R);
      }
    };
    FlatPos pp;                                            // where the range starts
    {
      pp.r = (int)(u_lo / T_total);
      const int f = (int)(u_lo - (long long)pp.r * T_total);
      int lo = 0, hi = n_dec;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pre[mid] <= f) lo = mid; else hi = mid;
      }
      pp.i = lo;
      pp.tt = f - pre[lo];
    }
    FlatPos cp = pp;
    const unsigned base = smem_u32(smem_raw);
    // what the producer knows about the entry it is in (looked up once per entry, not per tile)
    int p_i = -1, p_ctx = 0, p_lo0 = 0;
    const int* p_bt = nullptr;
    auto load_tile = [&](const FlatPos& p, int st) {
      if (p.i != p_i) {
        const int b = a.dec_seqs[p.i];
        p_i = p.i;
        p_ctx = a.context_lens[b];
        p_lo0 = a.window > 0 ? max(0, p_ctx - a.window) : 0;
        p_bt = a.block_tables + (size_t)b * a.bt_stride;
      }
      load_kv_tile<D>(a, p_bt, p.r / gchunks, p_lo0 + p.tt * MMA_BK, p_lo0, p_ctx, base + st * 2 * TILE_BYTES,
                      base + st * 2 * TILE_BYTES + TILE_BYTES, ps_log2);
    };
    load_tile(pp, 0);
    cp_async_commit();
    advance(pp);

    float m[2], l[2];
    float o[D / 8][4];
    unsigned qf[D / 16][4];
    int hi = 0, lo0 = 0, nrows = 0;
    bool fresh = true, from_first_tile = false;
    int* range_out = prefix_out + n_dec + 1;               // [pairs][2]: the CTAs with a pair's first and last piece
    const float sc = a.scale * LOG2E;
    for (int it = 0; it < ntiles; ++it) {
      if (it + 1 < ntiles) { load_tile(pp, (it + 1) % STAGES); advance(pp); }
      cp_async_commit();
      if (fresh) {
        // a new (token, kv head chunk): its queries, an empty softmax state
        const int b = a.dec_seqs[cp.i];
        const int t = a.cu_q_lens[b];
        hi = a.context_lens[b];
        lo0 = a.window > 0 ? max(0, hi - a.window) : 0;
        const int g0 = (cp.r % gchunks) * 16;
        nrows = min(16, G - g0);
        const __nv_bfloat16* qbase = (const __nv_bfloat16*)a.q + (size_t)t * a.q_stride + (size_t)((cp.r / gchunks) * G + g0) * D;
        const int nr = nrows;
        load_q_frags<D>(qf, [&](int r) { return r < nr ? qbase + (size_t)r * D : nullptr; });
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
        fresh = false;
        from_first_tile = cp.tt == 0;
      }
      cp_async_wait<STAGES - 1>();
      __syncthreads();
      const int st = it % STAGES;
      const unsigned ks = base + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
      const int key0 = warp * 16;                        // this warp's 16 keys of the tile
      const int tok0 = lo0 + cp.tt * MMA_BK + key0;
      if (tok0 < hi) {
        float s[2][4];
        qk_mma<D, 2>(qf, ks, key0, s);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int tk = tok0 + j * 8 + c2;
          s[j][0] = tk < hi ? s[j][0] * sc : -INFINITY;
          s[j][2] = tk < hi ? s[j][2] * sc : -INFINITY;
          s[j][1] = tk + 1 < hi ? s[j][1] * sc : -INFINITY;
          s[j][3] = tk + 1 < hi ? s[j][3] * sc : -INFINITY;
        }
        unsigned p[1][4];
        softmax_update<D, 2>(s, m, l, o, p);
        pv_mma<D, 2>(p, vs, key0, o);
      }
      __syncthreads();
      const bool last_of_entry = cp.tt + 1 == pre[cp.i + 1] - pre[cp.i];
      if (last_of_entry || it + 1 == ntiles) {
        // ---- this CTA's piece of the pair is complete: combine the four warps in the stage
        // just used and leave the piece in global memory
        l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
        l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
        l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
        l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
        float* co = reinterpret_cast<float*>(smem_raw + (size_t)st * 2 * TILE_BYTES);     // [4][16][D]
        if ((lane & 3) == 0) {
          cm[warp * 16 + g] = m[0]; cm[warp * 16 + g + 8] = m[1];
          cl[warp * 16 + g] = l[0]; cl[warp * 16 + g + 8] = l[1];
        }
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
          float* r0 = co + ((size_t)warp * 16 + g) * D + nt * 8 + c2;
          float* r1 = co + ((size_t)warp * 16 + g + 8) * D + nt * 8 + c2;
          r0[0] = o[nt][0]; r0[1] = o[nt][1];
          r1[0] = o[nt][2]; r1[1] = o[nt][3];
        }
        __syncthreads();
        const size_t pair = (size_t)cp.r * n_dec + cp.i, piece = pair + blockIdx.x;
        if (threadIdx.x == 0) {
          // the merge kernel finds a pair's pieces from these two, without the arithmetic of the ranges
          if (from_first_tile) range_out[2 * pair] = (int)blockIdx.x;
          if (last_of_entry) range_out[2 * pair + 1] = (int)blockIdx.x;
        }
        for (int e = threadIdx.x; e < nrows * D; e += MMA_THREADS) {
          const int r = e / D, col = e - r * D;
          const float M = fmaxf(fmaxf(cm[r], cm[16 + r]), fmaxf(cm[32 + r], cm[48 + r]));
          float L = 0.f, acc = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float mw = cm[w * 16 + r];
            if (mw != -INFINITY) {
              const float f = fast_exp2(mw - M);
              L += f * cl[w * 16 + r];
              acc += f * co[((size_t)w * 16 + r) * D + col];
            }
          }
          a.part_o[(piece * 16 + r) * D + col] = acc;
          if (col == 0) {
            a.part_ml[(piece * 16 + r) * 2] = M;
            a.part_ml[(piece * 16 + r) * 2 + 1] = L;
          }
        }
        __syncthreads();
        fresh = true;
      }
      advance(cp);
    }
    cp_async_wait<0>();
  }
  pdl_trigger();
}

// Merge of the pieces of attn_decode_flat_kernel: grid (n_dec, kv head chunks), a block merges
// the up to 16 heads of its chunk, a thread four neighbouring columns of a head.  The CTAs c
// with a piece of the pair are range[2 pair] .. range[2 pair + 1] (written by the CTAs that
// had the pair's first and last tile); CTA c left its piece at pair + c.  Everything a thread
// needs to find its pieces comes from loads that do not depend on one another, and the pieces
// of a pair are asked for four at a time before the first is used: the kernel is a few trips
// to L2 long, and that is all it is.
__global__ void __launch_bounds__(128) attn_merge_flat_kernel(AttnArgs a, int n_dec, int num_ctas,
                                                              const int* __restrict__ prefix) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x, r = blockIdx.y;
  const int b = a.dec_seqs[idx];
  if (b < 0) return;
  const int d = a.d, G = a.nh / a.nkv, gchunks = (G + 15) / 16, R = a.nkv * gchunks;
  const int kvh = r / gchunks, g0 = (r % gchunks) * 16, nrows = min(16, G - g0);
  const size_t q = (size_t)r * n_dec + idx;
  const int* range = prefix + n_dec + 1;
  const int tiles = prefix[idx + 1] - prefix[idx], T_total = prefix[n_dec];
  const int c_first = range[2 * q], c_last = range[2 * q + 1];
  __nv_bfloat16* out = (__nv_bfloat16*)a.out + (size_t)a.cu_q_lens[b] * a.nh * d + (size_t)(kvh * G + g0) * d;
  const int quads = d >> 2;
  if (tiles <= 0 || T_total <= 0) {
    for (int e = threadIdx.x; e < nrows * quads; e += blockDim.x) *reinterpret_cast<uint2*>(out + 4 * e) = make_uint2(0u, 0u);
    return;
  }
  // fewer tiles than CTAs: CTAs in between may have had nothing to do and left no piece
  const long long U = (long long)R * T_total, Gc = num_ctas;
  const bool gaps = U < Gc;
  for (int e = threadIdx.x; e < nrows * quads; e += blockDim.x) {
    const int row = e / quads, col = (e - row * quads) * 4;
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = c_first; c0 <= c_last; c0 += 4) {
      float2 ml[4];
      float4 po[4];
      bool have[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u;
        have[u] = c <= c_last && !(gaps && (c + 1) * U / Gc == c * U / Gc);
        if (have[u]) {
          ml[u] = *reinterpret_cast<const float2*>(a.part_ml + ((q + c) * 16 + row) * 2);
          po[u] = *reinterpret_cast<const float4*>(a.part_o + ((q + c) * 16 + row) * d + col);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (have[u] && ml[u].x != -INFINITY) {
          const float m_new = fmaxf(M, ml[u].x);
          const float f_old = fast_exp2(M - m_new), f = fast_exp2(ml[u].x - m_new);       // 2^-inf = 0
          L = L * f_old + f * ml[u].y;
          acc.x = acc.x * f_old + f * po[u].x;
          acc.y = acc.y * f_old + f * po[u].y;
          acc.z = acc.z * f_old + f * po[u].z;
          acc.w = acc.w * f_old + f * po[u].w;
          M = m_new;
        }
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint2 pk;
    pk.x = pack_bf16(acc.x * inv, acc.y * inv);
    pk.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + (size_t)row * d + col) = pk;
  }
}

// ---------------------------------------------------------------- prompt portions
template <int D>
__global__ void __launch_bounds__(MMA_THREADS) attn_prefill_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int TILE_BYTES = MMA_BK * D * 2;
  constexpr int STAGES = 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c2 = (lane & 3) * 2;
  // the lists that say what this CTA works on were copied in before the step began: they are
  // read while the kernel ahead (it writes the queries and the newest keys) is still finishing
  const int ps_log2 = 31 - __clz(a.page_size);
  const int b = a.tile_seq[blockIdx.x], q0 = a.tile_q0[blockIdx.x];
  const int h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int t0 = a.cu_q_lens[b], qlen = a.cu_q_lens[b + 1] - t0;
  const int ctx = a.context_lens[b];
  const int qstart = ctx - qlen;
  const int nrows = min(64, qlen - q0);
  const int first = qstart + q0;                     // position of the tile's first query
  const int hi = first + nrows;
  const int lo = a.window > 0 ? max(0, first - a.window + 1) : 0;
  const int kstart = (lo / MMA_BK) * MMA_BK;
  const int ntiles = (hi - kstart + MMA_BK - 1) / MMA_BK;
  const int* bt = a.block_tables + (size_t)b * a.bt_stride;
  const unsigned base = smem_u32(smem_raw);
  pdl_wait();

  load_kv_tile<D>(a, bt, kvh, kstart, lo, hi, base, base + TILE_BYTES, ps_log2);
  cp_async_commit();

  const int wrow0 = warp * 16;                       // this warp's rows of the tile
  const int pos0 = first + wrow0 + g, pos1 = pos0 + 8;   // positions of the thread's two rows
  unsigned qf[D / 16][4];
  const __nv_bfloat16* qbase = (const __nv_bfloat16*)a.q + (size_t)(t0 + q0 + wrow0) * a.q_stride + (size_t)h * D;
  load_q_frags<D>(qf, [&](int r) { return wrow0 + r < nrows ? qbase + (size_t)r * a.q_stride : nullptr; });
  const bool row0_ok = wrow0 + g < nrows, row1_ok = wrow0 + g + 8 < nrows;
  const int wlast = first + min(wrow0 + 15, nrows - 1);  // last position this warp needs

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
  const float sc = a.scale * LOG2E;

  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) {
      const int st = (it + 1) % STAGES;
      load_kv_tile<D>(a, bt, kvh, kstart + (it + 1) * MMA_BK, lo, hi, base + st * 2 * TILE_BYTES, base + st * 2 * TILE_BYTES + TILE_BYTES, ps_log2);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const int st = it % STAGES;
    const unsigned ks = base + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    const int kb = kstart + it * MMA_BK;
    if (wrow0 < nrows && kb <= wlast) {
      float s[8][4];
      qk_mma<D, 8>(qf, ks, 0, s);
      const bool interior = kb >= lo && kb + MMA_BK - 1 <= first + wrow0 &&
                            (a.window <= 0 || kb > wlast - a.window);
      if (interior) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j][0] *= sc; s[j][1] *= sc; s[j][2] *= sc; s[j][3] *= sc; }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tk = kb + j * 8 + c2 + (e & 1);
            const int pos = (e & 2) ? pos1 : pos0;
            const bool ok = ((e & 2) ? row1_ok : row0_ok) && tk >= lo && tk <= pos &&
                            (a.window <= 0 || tk > pos - a.window);
            s[j][e] = ok ? s[j][e] * sc : -INFINITY;
          }
        }
      }
      unsigned p[4][4];
      softmax_update<D, 8>(s, m, l, o, p);
      pv_mma<D, 8>(p, vs, 0, o);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  pdl_trigger();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const float inv0 = l[0] > 0.f ? 1.f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
  __nv_bfloat16* out = (__nv_bfloat16*)a.out;
  const size_t ostride = (size_t)a.nh * D;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + c2;
    if (row0_ok)
      *reinterpret_cast<unsigned*>(out + (size_t)(t0 + q0 + wrow0 + g) * ostride + (size_t)h * D + col) =
          pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
    if (row1_ok)
      *reinterpret_cast<unsigned*>(out + (size_t)(t0 + q0 + wrow0 + g + 8) * ostride + (size_t)h * D + col) =
          pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
  }
}

// ---------------------------------------------------------------- launchers
// (static and dynamic shared memory together count against the 48 KB that need no opt-in)
template <typename K> static int opt_in_smem(K kernel, size_t bytes, const char* who) {
  if (bytes > 32 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  return GG_OK;
}

// Launch with the slices of a (token, kv head) as one cluster, where the device can hold
// such clusters; the PDL attribute as in gg_launch.
template <typename K>
static cudaError_t launch_clustered(K kernel, dim3 grid, size_t smem, int cluster_z, cudaStream_t stream,
                                    const AttnArgs& a, int* max_clusters) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(MMA_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)cluster_z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (max_clusters) {
    cfg.numAttrs = 1;
    return cudaOccupancyMaxActiveClusters(max_clusters, kernel, &cfg);
  }
  cfg.numAttrs = gg_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

#define DECODE_STAGES 2
// The ring: 64 KB at d = 128, three CTAs per SM.  (A ring of six stages with one CTA per SM
// for launches that do not fill the device was measured: the attention itself no faster,
// the step slower, because the next kernel's CTAs found no room beside it.)
#define DECODE_STAGES_FEW 3       // for launches of at most two CTAs per SM: two tiles in flight per CTA
static size_t decode_ring_bytes(int d, int stages = DECODE_STAGES) { return (size_t)stages * 2 * MMA_BK * d * 2; }
// The inbox of the merge through the cluster: maxima and sums of every slice, and this
// CTA's share of every slice's rows.
static size_t decode_inbox_bytes(int d, int rows) { return (size_t)(ATTN_MAX_CLUSTER * 32 + rows * d + 2 * ATTN_MAX_CLUSTER) * sizeof(float); }

template <int D, int STAGES>
static int decode_cluster_capacity_of(int splits, int rows) {
  int n = 0;
  AttnArgs a = {};
  const size_t smem = decode_ring_bytes(D, STAGES) + decode_inbox_bytes(D, rows);
  cudaError_t e = cudaSuccess;
  if (smem > 32 * 1024)
    e = cudaFuncSetAttribute(attn_decode_mma_kernel<D, STAGES, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess)
    e = launch_clustered(attn_decode_mma_kernel<D, STAGES, true, false>, dim3(1, 1, splits), smem, splits, 0, a, &n);
  if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
  return n;
}

// How many clusters of `splits` decode CTAs the device holds at once (0: such clusters
// cannot be launched), with `group` query heads to a kv head (they size the merge's inbox).
// Asked once per head size, cluster size and inbox size.
static int decode_cluster_capacity(int d, int splits, int group, bool few) {
  static int cache[2][2][17][ATTN_MAX_CLUSTER + 1];
  static bool known[2][2][17][ATTN_MAX_CLUSTER + 1];
  if ((d != 64 && d != 128) || splits < 1 || splits > ATTN_MAX_CLUSTER || group < 1) return 0;
  const int di = d == 128, rows = group < 16 ? group : 16;
  if (!known[few][di][rows][splits]) {
    int n;
    if (few) n = d == 128 ? decode_cluster_capacity_of<128, DECODE_STAGES_FEW>(splits, rows) : decode_cluster_capacity_of<64, DECODE_STAGES_FEW>(splits, rows);
    else n = d == 128 ? decode_cluster_capacity_of<128, DECODE_STAGES>(splits, rows) : decode_cluster_capacity_of<64, DECODE_STAGES>(splits, rows);
    cache[few][di][rows][splits] = n;
    known[few][di][rows][splits] = true;
  }
  return cache[few][di][rows][splits];
}

int attn_decode_cluster_capacity(int d, int splits, int group) { return decode_cluster_capacity(d, splits, group, false); }

// *merged is set when the kernel wrote the final output itself (no merge kernel needed).
int attn_decode_mma(const AttnArgs& a, int n_dec, cudaStream_t stream, bool* merged) {
  GG_REQUIRE(power_of_two(a.page_size), "attn_decode: page size %d is not a power of two", a.page_size);
  const int G = a.nh / a.nkv, gchunks = (G + 15) / 16;
  GG_REQUIRE(a.nkv * gchunks <= 65535, "attn_decode: too many heads");
  dim3 grid(n_dec, a.nkv * gchunks, a.num_splits);
  const bool cluster = merged && a.num_splits <= ATTN_MAX_CLUSTER && attn_decode_cluster_capacity(a.d, a.num_splits, G) > 0;
  if (merged) *merged = cluster;
  // A launch that fits with two CTAs per SM gets a ring of three stages: each CTA then has two
  // tiles on their way, and a launch of so few CTAs is bound by how much is in flight (decode
  // steps at batch 1 and 16: 1.7 and 2.5 % faster; GOLLMGO_B200_DECODE_FEW=0 turns it off).
  static int num_sms = 0, few_ok = -1;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  if (few_ok < 0) { const char* ev = getenv("GOLLMGO_B200_DECODE_FEW"); few_ok = ev ? atoi(ev) : 1; }
  const long long groups = (long long)n_dec * a.nkv * gchunks;
  const bool few = few_ok && groups * a.num_splits <= 2LL * num_sms &&
                   (!cluster || groups * 10 <= 9LL * decode_cluster_capacity(a.d, a.num_splits, G, true));
  const size_t smem = decode_ring_bytes(a.d, few ? DECODE_STAGES_FEW : DECODE_STAGES) + (cluster ? decode_inbox_bytes(a.d, G < 16 ? G : 16) : 0);
  const bool rope = a.rope_inv_freq != nullptr;
  if (rope) {
    GG_REQUIRE(gchunks == 1, "attn_decode: the fused rotation takes at most 16 heads per kv head, not %d", G);
    GG_REQUIRE(a.rope_positions && (!a.rope_write_cache || a.slot_mapping), "attn_decode: fused rotation without positions or slots");
    GG_REQUIRE(a.q_stride % 8 == 0 && ((size_t)a.q % 16) == 0 && ((size_t)a.kcache % 16) == 0 && ((size_t)a.vcache % 16) == 0,
               "attn_decode: the fused rotation needs 16-byte aligned rows");
  }
  int rc;
  cudaError_t e;
#define DECODE_LAUNCH_ST(D_, ST_, CL_, RP_)                                                                  \
  do {                                                                                                       \
    if ((rc = opt_in_smem(attn_decode_mma_kernel<D_, ST_, CL_, RP_>, smem, "attn_decode"))) return rc;       \
    if (CL_) e = launch_clustered(attn_decode_mma_kernel<D_, ST_, CL_, RP_>, grid, smem, a.num_splits, stream, a, nullptr); \
    else e = gg_launch(attn_decode_mma_kernel<D_, ST_, CL_, RP_>, dim3(grid), dim3(MMA_THREADS), smem, stream, a); \
  } while (0)
#define DECODE_LAUNCH(D_, CL_, RP_)                                                                          \
  do {                                                                                                       \
    if (few) DECODE_LAUNCH_ST(D_, DECODE_STAGES_FEW, CL_, RP_);                                              \
    else DECODE_LAUNCH_ST(D_, DECODE_STAGES, CL_, RP_);                                                      \
  } while (0)
  if (a.d == 128) {
    if (cluster) { if (rope) DECODE_LAUNCH(128, true, true); else DECODE_LAUNCH(128, true, false); }
    else { if (rope) DECODE_LAUNCH(128, false, true); else DECODE_LAUNCH(128, false, false); }
  } else {
    if (cluster) { if (rope) DECODE_LAUNCH(64, true, true); else DECODE_LAUNCH(64, true, false); }
    else { if (rope) DECODE_LAUNCH(64, false, true); else DECODE_LAUNCH(64, false, false); }
  }
#undef DECODE_LAUNCH
#undef DECODE_LAUNCH_ST
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_decode_mma: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("attn_decode_mma");
}

int attn_prefill_mma(const AttnArgs& a, int num_tiles, cudaStream_t stream) {
  GG_REQUIRE(power_of_two(a.page_size), "attn_prefill: page size %d is not a power of two", a.page_size);
  GG_REQUIRE(num_tiles >= 0 && a.nh <= 65535, "attn_prefill: bad grid %d x %d", num_tiles, a.nh);
  if (num_tiles == 0) return GG_OK;
  dim3 grid(num_tiles, a.nh);
  int rc;
  if (a.d == 128) {
    const size_t smem = (size_t)2 * 2 * MMA_BK * 128 * 2;            // 64 KB
    if ((rc = opt_in_smem(attn_prefill_mma_kernel<128>, smem, "attn_prefill"))) return rc;
    gg_launch(attn_prefill_mma_kernel<128>, dim3(grid), dim3(MMA_THREADS), smem, stream, a);
  } else {
    const size_t smem = (size_t)2 * 2 * MMA_BK * 64 * 2;             // 32 KB
    gg_launch(attn_prefill_mma_kernel<64>, dim3(grid), dim3(MMA_THREADS), smem, stream, a);
  }
  return gg_check_launch("attn_prefill_mma");
}

// CTAs the flat decode kernel is launched with (its whole grid is resident at once).
int attn_decode_flat_ctas(int d) {
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  return (d == 128 ? 3 : 4) * num_sms;
}

// Scratch: part_o float[(n_dec * nkv * ceil(G / 16) + CTAs) * 16 * d], part_ml float[(same) * 16 * 2],
// prefix int[n_dec + 1 + 2 * n_dec * nkv * ceil(G / 16)] (the tiles before each token, then for each
// (kv head chunk, token) pair the CTAs with its first and its last piece).
int attn_decode_flat(const AttnArgs& a, int n_dec, int* prefix, cudaStream_t stream) {
  GG_REQUIRE(power_of_two(a.page_size), "attn_decode: page size %d is not a power of two", a.page_size);
  GG_REQUIRE(n_dec <= FLAT_MAX_SEQS, "attn_decode: %d decoded tokens; the flat kernel takes at most %d", n_dec, FLAT_MAX_SEQS);
  GG_REQUIRE(prefix != nullptr, "attn_decode: no prefix scratch given");
  const int ctas = attn_decode_flat_ctas(a.d);
  const size_t smem = decode_ring_bytes(a.d);
  int rc;
  cudaError_t e;
  if (a.d == 128) {
    if ((rc = opt_in_smem(attn_decode_flat_kernel<128>, smem, "attn_decode"))) return rc;
    e = gg_launch(attn_decode_flat_kernel<128>, dim3(ctas), dim3(MMA_THREADS), smem, stream, a, n_dec, prefix);
  } else {
    e = gg_launch(attn_decode_flat_kernel<64>, dim3(ctas), dim3(MMA_THREADS), smem, stream, a, n_dec, prefix);
  }
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_decode_flat: launch: %s", cudaGetErrorString(e));
  if ((rc = gg_check_launch("attn_decode_flat"))) return rc;
  const int G = a.nh / a.nkv, R = a.nkv * ((G + 15) / 16);
  GG_REQUIRE(R <= 65535, "attn_decode_flat: too many heads");
  e = gg_launch(attn_merge_flat_kernel, dim3(n_dec, R), dim3(128), 0, stream, a, n_dec, ctas, (const int*)prefix);
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_merge_flat: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("attn_merge_flat");
}
