// Matrix products for a few dozen tokens (decode steps of 17 to 64 sequences, short prompt
// portions) on the fifth-generation tensor cores: out[M, N] = x[M, K] W[N, K]^T, bfloat16 in,
// float32 accumulation in tensor memory.
//
// With so few tokens the product is one pass over the weights, as in gemm_small_m.cu, but the
// tokens no longer fit one warp's registers.  Here the operands are swapped: 128 rows of W
// are the M side of tcgen05.mma and the (padded) tokens its N side, so a CTA streams a
// [128 x K] slab of W through shared memory once and the small x tile rides along:
//   warp 0  one lane issues the TMA loads per stage: a 128 x 64 tile of W (two 64-row boxes,
//           gate and up rows, in the gated mode) and an NP x 64 tile of x, four stages deep.
//           The loads of W for the first stages are issued before griddepcontrol.wait: the
//           weights do not depend on the kernel before this one, only x does.
//   warp 1  allocates NP columns of tensor memory; one lane issues tcgen05.mma (M = 128,
//           N = NP, K = 16; four per stage) and releases each stage with tcgen05.commit.
//   warps 2-5  read the accumulator with tcgen05.ld (a warp its 32 lanes = 32 rows of W) and
//           leave it in shared memory as float32 [token][row].
// Few row slabs would leave most SMs without work (N = 4096 gives 32), so K is split over
// the 1, 2, 4 or 8 CTAs of a thread-block cluster; after a cluster barrier every CTA sums
// its share of the rows over all CTAs' partial results through distributed shared memory,
// in a fixed order (no atomics), applies the epilogue and stores.
// Epilogues: bfloat16; float32; SiLU-gated: rows 0-63 of the slab are gate rows and rows
// 64-127 the up rows of the same 64 features (formula: kernels/gollmgo_ops.cu:361-374).
// Every wait on an mbarrier is bounded and reports through *status; the barriers of the
// cluster are reached by every thread whatever its waits returned.  No TMA load uses
// cluster multicast.
#include "tc_common.cuh"

#define MM_BK 64
#define MM_STAGES 4
#define MM_THREADS 192
#define MM_W_BYTES (128 * MM_BK * 2)

enum { MM_OUT_BF16 = 0, MM_OUT_F32 = 1, MM_OUT_SILU = 2 };
enum { MM_ERR_EMPTY_WAIT = 41, MM_ERR_FULL_WAIT = 42, MM_ERR_ACC_WAIT = 43, MM_ERR_DRAIN = 44 };

__device__ __forceinline__ unsigned mm_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void mm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float mm_ld_cluster(unsigned local_addr, unsigned rank) {
  float v;
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %1, %2;\n\t"
      "ld.shared::cluster.f32 %0, [ra];\n\t}"
      : "=f"(v) : "r"(local_addr), "r"(rank) : "memory");
  return v;
}

// grid (S, slabs), cluster (S, 1, 1): CTA (s, t) multiplies slab t over its share of K.
template <int MODE, int NP>
__global__ void __launch_bounds__(MM_THREADS)
gemm_mid_m_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  void* __restrict__ out, int M, int N, int K, int* __restrict__ status) {
  constexpr unsigned X_BYTES = NP * MM_BK * 2, STAGE_BYTES = MM_W_BYTES + X_BYTES;
  extern __shared__ unsigned char mm_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * MM_STAGES + 1];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles = (tc_smem(mm_smem_raw) + 1023u) & ~1023u;        // 1024-byte aligned stages
  unsigned char* tiles_ptr = mm_smem_raw + (tiles - tc_smem(mm_smem_raw));
  const unsigned full0 = tc_smem(&bars[0]), empty0 = tc_smem(&bars[MM_STAGES]), acc_full = tc_smem(&bars[2 * MM_STAGES]);
  const int S = gridDim.x, rank = (int)mm_cluster_rank();
  const int slab = blockIdx.y;
  const int num_kb = (K + MM_BK - 1) / MM_BK;
  const int kb0 = (int)((long long)rank * num_kb / S), kb1 = (int)((long long)(rank + 1) * num_kb / S);
  const int my_kb = kb1 - kb0;
  // rows of W in this slab: 128 outputs, or 64 gated features (gate rows n0.., up rows N + n0..)
  const int n0 = MODE == MM_OUT_SILU ? slab * 64 : slab * 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MM_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(acc_full, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"((unsigned)NP) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_base_s;
  pdl_trigger();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    auto load_w = [&](int i) {
      const int s = i % MM_STAGES;
      const unsigned dst = tiles + s * STAGE_BYTES, bar = full0 + 8 * s;
      const int k = (kb0 + i) * MM_BK;
      if (MODE == MM_OUT_SILU) {
        tma_load_2d(dst, &map_w, k, n0, bar);                            // 64 gate rows
        tma_load_2d(dst + MM_W_BYTES / 2, &map_w, k, N + n0, bar);       // 64 up rows
      } else {
        tma_load_2d(dst, &map_w, k, n0, bar);
      }
    };
    auto load_x = [&](int i) {
      const int s = i % MM_STAGES;
      tma_load_2d(tiles + s * STAGE_BYTES + MM_W_BYTES, &map_x, (kb0 + i) * MM_BK, 0, full0 + 8 * s);
    };
    // the weights of the first stages, before the kernel ahead has finished; then its output
    const int early = min(MM_STAGES, my_kb);
    for (int i = 0; i < early; ++i) { mbar_expect_tx(full0 + 8 * i, STAGE_BYTES); load_w(i); }
    pdl_wait();
    for (int i = 0; i < early; ++i) load_x(i);
    int issued = early;
    for (int i = early; i < my_kb; ++i) {
      const int s = i % MM_STAGES;
      if (!mbar_wait(empty0 + 8 * s, ((i / MM_STAGES) & 1) ^ 1)) { atomicExch(status, MM_ERR_EMPTY_WAIT); atomicExch(&abort_s, 1); break; }
      if (*(volatile int*)&abort_s) break;
      mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
      load_w(i);
      load_x(i);
      issued = i + 1;
    }
    // on an abort: let the copies that were issued land before shared memory is reused
    if (*(volatile int*)&abort_s) {
      for (int i = max(0, issued - MM_STAGES); i < issued; ++i)
        if (!mbar_wait(full0 + 8 * (i % MM_STAGES), (i / MM_STAGES) & 1)) { atomicExch(status, MM_ERR_DRAIN); break; }
    }
  } else {
    pdl_wait();
    if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer: A = the slab of W (M = 128), B = the tokens (N = NP), both K-major
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NP >> 3) << 17) | ((128u >> 4) << 24);
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % MM_STAGES;
        if (*(volatile int*)&abort_s) break;
        if (!mbar_wait(full0 + 8 * s, (i / MM_STAGES) & 1)) { atomicExch(status, MM_ERR_FULL_WAIT); atomicExch(&abort_s, 1); break; }
        tc_fence_after();
        const unsigned long long a_desc = tc_smem_desc(tiles + s * STAGE_BYTES);
        const unsigned long long b_desc = tc_smem_desc(tiles + s * STAGE_BYTES + MM_W_BYTES);
#pragma unroll
        for (int k = 0; k < MM_BK / 16; ++k)
          tc_mma(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty0 + 8 * s);
      }
      tc_commit(acc_full);                           // the accumulator is complete (also on abort)
    }
  }
  // ---------------- accumulator -> shared memory as float32 [token][row], over the stages
  float* dump = reinterpret_cast<float*>(tiles_ptr);                     // [NP][128]
  if (warp >= 2) {
    const int quarter = warp & 3, row = quarter * 32 + lane;
    bool ok = mbar_wait(acc_full, 0);
    if (!ok) { atomicExch(status, MM_ERR_ACC_WAIT); atomicExch(&abort_s, 1); }
    tc_fence_after();
    if (ok && !*(volatile int*)&abort_s) {
#pragma unroll
      for (int c = 0; c < NP; c += 32) {
        unsigned v[32];
        if (my_kb > 0) {
          tc_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;      // no share of K: nothing was accumulated
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) dump[(c + j) * 128 + row] = __uint_as_float(v[j]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  mm_cluster_sync();                                 // every CTA's partial result is in its shared memory
  // ---------------- this CTA's share of the rows, summed over the cluster in rank order
  {
    const unsigned dump_a = tc_smem(dump);
    if (MODE == MM_OUT_SILU) {
      const int per = 64 / S, f_lo = rank * per;     // features of the slab this CTA finishes
      for (int e = threadIdx.x; e < per * M; e += MM_THREADS) {
        const int t = e / per, f = f_lo + (e - t * per);
        float gate = 0.f, up = 0.f;
        for (int p = 0; p < S; ++p) {
          gate += mm_ld_cluster(dump_a + (unsigned)((t * 128 + f) * 4), p);
          up += mm_ld_cluster(dump_a + (unsigned)((t * 128 + 64 + f) * 4), p);
        }
        const int n = n0 + f;
        if (n < N)
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)t * N + n] = __float2bfloat16_rn(gate / (1.f + __expf(-gate)) * up);
      }
    } else {
      const int per = 128 / S, r_lo = rank * per;
      for (int e = threadIdx.x; e < per * M; e += MM_THREADS) {
        const int t = e / per, r = r_lo + (e - t * per);
        float v = 0.f;
        for (int p = 0; p < S; ++p) v += mm_ld_cluster(dump_a + (unsigned)((t * 128 + r) * 4), p);
        const int n = n0 + r;
        if (n < N) {
          if (MODE == MM_OUT_F32) reinterpret_cast<float*>(out)[(size_t)t * N + n] = v;
          else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)t * N + n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
  mm_cluster_sync();                                 // nobody leaves while a neighbour may still read it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)NP) : "memory");
  }
}

// ---------------------------------------------------------------- host side
template <typename Kern>
static cudaError_t mm_launch(Kern kernel, dim3 grid, size_t smem, int cluster_x, cudaStream_t stream,
                             const CUtensorMap& map_x, const CUtensorMap& map_w, void* out, int M, int N, int K,
                             int* status) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(MM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gg_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, map_x, map_w, out, M, N, K, status);
}

// mode: 0 = bfloat16 out [M, N]; 1 = float32 out [M, N]; 2 = W is [2N, K] (gate rows then up
// rows), out is bfloat16 [M, N] = silu(x Wg^T) * (x Wu^T).  1 <= M <= 64.  status: one int in
// device memory, left untouched unless a wait inside the kernel ran out (then non-zero).
extern "C" int gg_gemm_mid_m(const void* x, long long ldx, const void* W, void* out, int M, int N, int K,
                             int mode, int* status, cudaStream_t stream) {
  GG_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_mid_m: bad sizes M=%d N=%d K=%d", M, N, K);
  GG_REQUIRE(M <= 64, "gemm_mid_m: %d tokens; this kernel takes at most 64", M);
  GG_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_mid_m: K=%d and the row stride %lld of x must be multiples of 8", K, ldx);
  GG_REQUIRE(((size_t)x % 16) == 0 && ((size_t)W % 16) == 0, "gemm_mid_m: x and W must be 16-byte aligned");
  GG_REQUIRE(mode >= 0 && mode <= 2, "gemm_mid_m: unknown mode %d", mode);
  GG_REQUIRE(status != nullptr, "gemm_mid_m: no status word given");
  if (M == 0) return GG_OK;
  const int np = M <= 32 ? 32 : 64;
  CUtensorMap map_x, map_w;
  int rc = gg_make_map_2d(&map_x, x, M, K, ldx, np);
  if (rc) return rc;
  const int w_rows = mode == MM_OUT_SILU ? 2 * N : N;
  rc = gg_make_map_2d(&map_w, W, w_rows, K, K, mode == MM_OUT_SILU ? 64 : 128);
  if (rc) return rc;
  const int slabs = mode == MM_OUT_SILU ? (N + 63) / 64 : (N + 127) / 128;
  GG_REQUIRE(slabs <= 65535, "gemm_mid_m: too many row slabs (%d)", slabs);
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  // split K over as many CTAs of a cluster as still fit the machine at once (two CTAs per SM)
  const int num_kb = (K + MM_BK - 1) / MM_BK;
  int S = 1;
  while (S < 8 && slabs * (S * 2) <= 2 * num_sms && S * 2 <= num_kb) S *= 2;
  const size_t smem = (size_t)MM_STAGES * (MM_W_BYTES + (size_t)np * MM_BK * 2) + 1024;
  dim3 grid(S, slabs);
  cudaError_t e = cudaSuccess;
#define MM_LAUNCH(MODE, NP)                                                                                \
  do {                                                                                                     \
    static bool set = false;                                                                               \
    if (!set) {                                                                                            \
      e = cudaFuncSetAttribute(gemm_mid_m_kernel<MODE, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_mid_m: %s", cudaGetErrorString(e));          \
      set = true;                                                                                          \
    }                                                                                                      \
    e = mm_launch(gemm_mid_m_kernel<MODE, NP>, grid, smem, S, stream, map_x, map_w, out, M, N, K, status); \
  } while (0)
  if (np == 32) {
    if (mode == MM_OUT_BF16) MM_LAUNCH(MM_OUT_BF16, 32); else if (mode == MM_OUT_F32) MM_LAUNCH(MM_OUT_F32, 32); else MM_LAUNCH(MM_OUT_SILU, 32);
  } else {
    if (mode == MM_OUT_BF16) MM_LAUNCH(MM_OUT_BF16, 64); else if (mode == MM_OUT_F32) MM_LAUNCH(MM_OUT_F32, 64); else MM_LAUNCH(MM_OUT_SILU, 64);
  }
#undef MM_LAUNCH
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_mid_m: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("gemm_mid_m");
}
