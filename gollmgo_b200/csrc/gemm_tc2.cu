// The tcgen05 matrix product with CTA pairs (cta_group::2): two CTAs of a cluster, on two SMs,
// work on one 256 x 256 output tile.  Each CTA loads its own 128 rows of x and its own 128 rows
// of W per stage (so each SM moves 32 KB per 64 values of k instead of the 48 KB of the
// one-CTA kernel in gemm_tc.cu); the even CTA issues tcgen05.mma.cta_group::2 (M = 256,
// N = 256, K = 16), which reads both CTAs' shared memory and writes each CTA's own 128 rows of
// the accumulator into that CTA's tensor memory.
//
//   * TMA loads are the cta_group::2 form, without multicast: both CTAs load into their own
//     shared memory and both signal the EVEN CTA's "full" mbarrier (same offset, peer bit
//     cleared), which expects the bytes of all four boxes.
//   * tcgen05.commit.cta_group::2 with a CTA mask of 0b11 releases a stage in both CTAs, and
//     at the end of a tile tells both CTAs' epilogue warps that the accumulator is complete.
//   * The epilogue warps of both CTAs hand an accumulator buffer back by arriving on the even
//     CTA's barrier (the odd CTA through its cluster address).
//   * The pair is persistent: pair p takes tiles p, p + pairs, ...; two accumulators of 256
//     columns in each CTA's tensor memory let one tile's epilogue overlap the next tile's MMAs.
// Gated mode: columns [0,128) of the tile are gate features (the even CTA's rows of W) and
// [128,256) the up features of the same 128 features (the odd CTA's), so each CTA's epilogue
// has both for its rows.
// All mbarrier waits are bounded and report through *status; the cluster barriers at the start
// and the end are reached by every thread whatever its waits returned.
#include "tc_common.cuh"

#define T2_BK 64
#define T2_STAGES 6
#define T2_THREADS 192
#define T2_PEER_MASK 0xFEFFFFFFu      // clears the bit that tells the two CTAs' shared windows apart

enum { T2_OUT_BF16 = 0, T2_OUT_F32 = 1, T2_OUT_SILU = 2 };
enum { T2_ERR_EMPTY_WAIT = 21, T2_ERR_FULL_WAIT = 22, T2_ERR_ACC_WAIT = 23, T2_ERR_DRAIN = 24 };

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                            unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
        "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// Arrive on the barrier at the same offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
// Arrive on the barrier at this offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar, unsigned rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(bar), "r"(rank) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(T2_THREADS)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                void* __restrict__ out, int M, int N, int K, int tiles_m, int num_tiles,
                int* __restrict__ status) {
  constexpr int BN = 256;
  constexpr unsigned A_BYTES = 128 * T2_BK * 2, B_BYTES = 128 * T2_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ unsigned char t2_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * T2_STAGES + 4];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const unsigned tiles = (tc_smem(t2_smem_raw) + 1023u) & ~1023u;
  const unsigned full0 = tc_smem(&bars[0]), empty0 = tc_smem(&bars[T2_STAGES]);
  const unsigned acc_full0 = tc_smem(&bars[2 * T2_STAGES]), acc_empty0 = tc_smem(&bars[2 * T2_STAGES + 2]);
  const int n_out_tile = MODE == T2_OUT_SILU ? 128 : BN;
  const int num_kb = (K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"(2u * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // the partner's barriers exist before anything signals them
  tc_fence_after();
  const unsigned tmem_base = tmem_base_s;
  pdl_trigger();
  pdl_wait();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer (one per CTA): own rows of x, own rows of W
    int issued = 0, it = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs) {
      const int m0 = (t % tiles_m) * 256 + (int)rank * 128;
      const int nt0 = (t / tiles_m) * n_out_tile;
      const int w_row = MODE == T2_OUT_SILU ? (rank == 0 ? nt0 : N + nt0) : nt0 + (int)rank * 128;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % T2_STAGES;
        const unsigned phase = (it / T2_STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, phase ^ 1)) { atomicExch(status, T2_ERR_EMPTY_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
        if (*(volatile int*)&abort_s) { ok = false; break; }
        const unsigned a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
        const unsigned full_even = (full0 + 8 * s) & T2_PEER_MASK;         // the even CTA's barrier
        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);      // four boxes: two from each CTA
        tma_load_2d_pair(a_dst, &map_x, kb * T2_BK, m0, full_even);
        tma_load_2d_pair(b_dst, &map_w, kb * T2_BK, w_row, full_even);
        issued = it + 1;
      }
    }
    if (*(volatile int*)&abort_s && rank == 0) {
      for (int i = max(0, issued - T2_STAGES); i < issued; ++i)
        if (!mbar_wait(full0 + 8 * (i % T2_STAGES), (i / T2_STAGES) & 1)) { atomicExch(status, T2_ERR_DRAIN); break; }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer: the even CTA, for the pair.  M = 256, N = 256.
    const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((256u >> 4) << 24);
    bool ok = true;
    int it = 0, local = 0;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++local) {
      const int buf = local & 1;
      if (!mbar_wait(acc_empty0 + 8 * buf, ((local >> 1) & 1) ^ 1)) { atomicExch(status, T2_ERR_ACC_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
      tc_fence_after();
      const unsigned d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % T2_STAGES;
        const unsigned phase = (it / T2_STAGES) & 1;
        if (*(volatile int*)&abort_s) { ok = false; break; }
        if (!mbar_wait(full0 + 8 * s, phase)) { atomicExch(status, T2_ERR_FULL_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
        tc_fence_after();
        const unsigned long long a_desc = tc_smem_desc(tiles + s * STAGE_BYTES);
        const unsigned long long b_desc = tc_smem_desc(tiles + s * STAGE_BYTES + A_BYTES);
#pragma unroll
        for (int k = 0; k < T2_BK / 16; ++k)
          tc_mma_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit_pair(empty0 + 8 * s);               // the stage is free in both CTAs
      }
      tc_commit_pair(acc_full0 + 8 * buf);            // both CTAs' accumulators are complete
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: each CTA drains its own 128 rows
    const int quarter = warp & 3;
    int local = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++local) {
      const int buf = local & 1;
      const int m0 = (t % tiles_m) * 256 + (int)rank * 128, n0 = (t / tiles_m) * n_out_tile;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(acc_full0 + 8 * buf, (local >> 1) & 1)) { atomicExch(status, T2_ERR_ACC_WAIT); atomicExch(&abort_s, 1); break; }
      if (*(volatile int*)&abort_s) break;
      tc_fence_after();
      const unsigned tlane = tmem_base + buf * BN + ((unsigned)(quarter * 32) << 16);
      if (MODE == T2_OUT_SILU) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + n0;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          unsigned g[32], u[32];
          tc_load32(tlane + c, g);
          tc_load32(tlane + 128 + c, u);
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float gj = __uint_as_float(g[j]);
            v[j] = gj / (1.f + __expf(-gj)) * __uint_as_float(u[j]);
          }
          if (row < M) store_row32(o + c, v, N - (n0 + c));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          unsigned r[32];
          tc_load32(tlane + c, r);
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (row < M) {
            if (MODE == T2_OUT_F32) store_row32(reinterpret_cast<float*>(out) + (size_t)row * N + n0 + c, v, N - (n0 + c));
            else store_row32(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + n0 + c, v, N - (n0 + c));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8 * buf, 0);       // the even CTA's barrier counts all eight warps
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // nobody leaves while the partner may still read or signal here
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * BN) : "memory");
  }
}

// Same contract as gg_gemm_tc (mode 0 bf16, 1 f32, 2 SiLU-gated with W = [2N, K]); CTA pairs.
extern "C" int gg_gemm_tc2(const void* x, long long ldx, const void* W, void* out, int M, int N, int K,
                           int mode, int* status, cudaStream_t stream) {
  GG_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc2: bad sizes M=%d N=%d K=%d", M, N, K);
  GG_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_tc2: K=%d and the row stride %lld of x must be multiples of 8", K, ldx);
  GG_REQUIRE(((size_t)x % 16) == 0 && ((size_t)W % 16) == 0, "gemm_tc2: x and W must be 16-byte aligned");
  GG_REQUIRE(mode >= 0 && mode <= 2, "gemm_tc2: unknown mode %d", mode);
  GG_REQUIRE(N % 2 == 0 || mode == T2_OUT_F32, "gemm_tc2: bfloat16 rows of odd length are not 4-byte aligned");
  GG_REQUIRE(status != nullptr, "gemm_tc2: no status word given");
  if (M == 0) return GG_OK;
  CUtensorMap map_x, map_w;
  int rc = gg_make_map_2d(&map_x, x, M, K, ldx, 128);
  if (rc) return rc;
  rc = gg_make_map_2d(&map_w, W, mode == T2_OUT_SILU ? 2 * N : N, K, K, 128);
  if (rc) return rc;
  const int n_tile = mode == T2_OUT_SILU ? 128 : 256;
  const int tiles_m = (M + 255) / 256, tiles_n = (N + n_tile - 1) / n_tile;
  const long long num_tiles_ll = (long long)tiles_m * tiles_n;
  GG_REQUIRE(num_tiles_ll < (1ll << 30), "gemm_tc2: too many tiles");
  const int num_tiles = (int)num_tiles_ll;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  const int pairs = num_tiles < num_sms / 2 ? num_tiles : num_sms / 2;
  const size_t smem = (size_t)T2_STAGES * (128 * T2_BK * 2 * 2) + 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(T2_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gg_pdl_enabled() ? 2 : 1;
  cudaError_t e;
#define T2_LAUNCH(MODE)                                                                                     \
  do {                                                                                                      \
    static bool set = false;                                                                                \
    if (!set) {                                                                                             \
      e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_tc2: %s", cudaGetErrorString(e));             \
      set = true;                                                                                           \
    }                                                                                                       \
    e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE>, map_x, map_w, out, M, N, K, tiles_m, num_tiles, status); \
  } while (0)
  if (mode == T2_OUT_BF16) T2_LAUNCH(T2_OUT_BF16);
  else if (mode == T2_OUT_F32) T2_LAUNCH(T2_OUT_F32);
  else T2_LAUNCH(T2_OUT_SILU);
#undef T2_LAUNCH
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_tc2: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("gemm_tc2");
}
