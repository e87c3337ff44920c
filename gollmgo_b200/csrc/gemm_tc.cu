// Matrix products for many tokens (prompt portions) on the fifth-generation tensor
// cores: out[M, N] = x[M, K] W[N, K]^T, bfloat16 in, float32 accumulation in tensor
// memory.  Both operands are K-major, as the activations and the checkpoint's weights
// already are, so no transposed copies exist anywhere.
//
// A persistent CTA (one per SM) computes 128 x BN tiles (BN = 256, or 128 gate + 128 up
// rows for the gated product), one after the other, with six warps in three roles:
//   warp 0  one lane issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//           of a 128 x 64 tile of x and a BN x 64 tile of W per stage, four stages
//           deep, each landing on an mbarrier with a byte count;
//   warp 1  allocates 2 x BN columns of tensor memory (two accumulators, so that one
//           tile's epilogue overlaps the next tile's products); one lane issues tcgen05.mma
//           (M = 128, N = BN, K = 16; four per stage) from shared-memory descriptors
//           and releases each stage with tcgen05.commit;
//   warps 2-5  wait for the last commit, read the accumulator with tcgen05.ld (each
//           warp its own 32 lanes = 32 rows of the tile), apply the epilogue and
//           store.
// Epilogues: bfloat16; float32; SiLU-gated: columns [0,128) of the accumulator come
// from the gate rows of W and [128,256) from the up rows of the same features, and
// the tile written is silu(gate) * up (formula: kernels/gollmgo_ops.cu:361-374).
// Rows of x beyond M, rows of W beyond N and columns beyond K are zero-filled by TMA;
// the epilogue only stores what lies inside the output.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a code in
// *status, and the CTA stops issuing work, gives up its tensor memory and returns; the
// host treats a non-zero status as an error.  No TMA load uses cluster multicast.
#include "tc_common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_STAGES 4
#define TC_THREADS 192
enum { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_SILU = 2 };
enum { TC_ERR_EMPTY_WAIT = 1, TC_ERR_FULL_WAIT = 2, TC_ERR_ACC_WAIT = 3, TC_ERR_DRAIN = 4 };

// A persistent CTA walks over output tiles blockIdx.x, blockIdx.x + gridDim.x, ...; tile t is
// (row block t % tiles_m, column block t / tiles_m), so CTAs that run together share a block of
// W.  The accumulator is double-buffered in tensor memory (2 x 256 columns): while the
// epilogue warps drain one buffer the MMA warp fills the other.
template <int MODE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ out, int M, int N, int K, int tiles_m, int num_tiles,
               int* __restrict__ status, int withhold_loads) {
  constexpr int BN = 256;
  constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * TC_STAGES + 4];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles = (tc_smem(tc_smem_raw) + 1023u) & ~1023u;        // 1024-byte aligned stages
  const unsigned full0 = tc_smem(&bars[0]), empty0 = tc_smem(&bars[TC_STAGES]);
  const unsigned acc_full0 = tc_smem(&bars[2 * TC_STAGES]), acc_empty0 = tc_smem(&bars[2 * TC_STAGES + 2]);
  // output tile: in the gated mode N counts gated features and a tile has 128 of them
  const int n_out_tile = MODE == TC_OUT_SILU ? 128 : BN;
  const int num_kb = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 4); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"(2u * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_base_s;
  pdl_trigger();
  pdl_wait();                                   // x is the previous kernel's output

  if (warp == 0 && lane == 0 && !withhold_loads) {
    // ---------------- TMA producer (withhold_loads: the self-test of the bounded waits; nothing is
    // loaded, so the consumers' waits must run out, report, and let the CTA return)
    int issued = 0, it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m0 = (t % tiles_m) * TC_BM, n0 = (t / tiles_m) * n_out_tile;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % TC_STAGES;
        const unsigned phase = (it / TC_STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, phase ^ 1)) { atomicExch(status, TC_ERR_EMPTY_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
        if (*(volatile int*)&abort_s) { ok = false; break; }
        const unsigned a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        tma_load_2d(a_dst, &map_x, kb * TC_BK, m0, full0 + 8 * s);
        if (MODE == TC_OUT_SILU) {
          tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, full0 + 8 * s);                      // 128 gate rows
          tma_load_2d(b_dst + B_BYTES / 2, &map_w, kb * TC_BK, N + n0, full0 + 8 * s);    // 128 up rows
        } else {
          tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, full0 + 8 * s);
        }
        issued = it + 1;
      }
    }
    // on an abort: let the copies that were issued land before shared memory is given up
    if (*(volatile int*)&abort_s) {
      for (int i = max(0, issued - TC_STAGES); i < issued; ++i)
        if (!mbar_wait(full0 + 8 * (i % TC_STAGES), (i / TC_STAGES) & 1)) { atomicExch(status, TC_ERR_DRAIN); break; }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
    const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
    bool ok = true;
    int it = 0, local = 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
      const int buf = local & 1;
      // the epilogue must have drained this buffer (two tiles ago)
      if (!mbar_wait(acc_empty0 + 8 * buf, ((local >> 1) & 1) ^ 1)) { atomicExch(status, TC_ERR_ACC_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
      tc_fence_after();
      const unsigned d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % TC_STAGES;
        const unsigned phase = (it / TC_STAGES) & 1;
        if (*(volatile int*)&abort_s) { ok = false; break; }
        if (!mbar_wait(full0 + 8 * s, phase)) { atomicExch(status, TC_ERR_FULL_WAIT); atomicExch(&abort_s, 1); ok = false; break; }
        tc_fence_after();
        const unsigned long long a_desc = tc_smem_desc(tiles + s * STAGE_BYTES);
        const unsigned long long b_desc = tc_smem_desc(tiles + s * STAGE_BYTES + A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)          // 16 values of k = 32 bytes = 2 units of 16 bytes
          tc_mma(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty0 + 8 * s);                    // the stage is free once these MMAs have read it
      }
      tc_commit(acc_full0 + 8 * buf);                 // this tile's accumulator is complete (also on abort)
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +32
    const int quarter = warp & 3;
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (t % tiles_m) * TC_BM, n0 = (t / tiles_m) * n_out_tile;
      const int row = m0 + quarter * 32 + lane;
      if (!mbar_wait(acc_full0 + 8 * buf, (local >> 1) & 1)) { atomicExch(status, TC_ERR_ACC_WAIT); atomicExch(&abort_s, 1); break; }
      if (*(volatile int*)&abort_s) break;
      tc_fence_after();
      const unsigned tlane = tmem_base + buf * BN + ((unsigned)(quarter * 32) << 16);
      if (MODE == TC_OUT_SILU) {
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
            if (MODE == TC_OUT_F32) store_row32(reinterpret_cast<float*>(out) + (size_t)row * N + n0 + c, v, N - (n0 + c));
            else store_row32(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + n0 + c, v, N - (n0 + c));
          }
        }
      }
      // hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * BN) : "memory");
  }
}

// ---------------------------------------------------------------- host side
GgEncodeTiledFn gg_encode_tiled() {
  static GgEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (GgEncodeTiledFn)p;
  }
  return fn;
}

// Tensor map of a row-major bf16 matrix [rows, cols] with row stride ld (elements), boxes of
// box_rows x 64 columns, 128-byte swizzle, zero fill outside.
int gg_make_map_2d(CUtensorMap* map, const void* ptr, int rows, int cols, long long ld, int box_rows) {
  GgEncodeTiledFn fn = gg_encode_tiled();
  if (!fn) return gg_fail(GG_ERR_CUDA, "gemm_tc: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gg_fail(GG_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return GG_OK;
}

// mode: 0 = bfloat16 out [M, N]; 1 = float32 out [M, N]; 2 = W is [2N, K] (gate rows then up
// rows), out is bfloat16 [M, N] = silu(x Wg^T) * (x Wu^T).  status: one int in device memory,
// left untouched unless a wait inside the kernel ran out (then non-zero).
static int gemm_tc_launch(const void* x, long long ldx, const void* W, void* out, int M, int N, int K,
                          int mode, int* status, int withhold_loads, cudaStream_t stream);

extern "C" int gg_gemm_tc(const void* x, long long ldx, const void* W, void* out, int M, int N, int K,
                          int mode, int* status, cudaStream_t stream) {
  return gemm_tc_launch(x, ldx, W, out, M, N, K, mode, status, 0, stream);
}

// Self-test of the bounded waits: the same launch, but the loads are withheld, so no barrier a
// consumer waits on ever completes.  The kernel must set *status non-zero and return within a
// few seconds, leaving the context usable.  out is not written.
extern "C" int gg_gemm_tc_withheld(const void* x, long long ldx, const void* W, void* out, int M, int N,
                                   int K, int* status, cudaStream_t stream) {
  return gemm_tc_launch(x, ldx, W, out, M, N, K, TC_OUT_BF16, status, 1, stream);
}

static int gemm_tc_launch(const void* x, long long ldx, const void* W, void* out, int M, int N, int K,
                          int mode, int* status, int withhold_loads, cudaStream_t stream) {
  GG_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  GG_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_tc: K=%d and the row stride %lld of x must be multiples of 8", K, ldx);
  GG_REQUIRE(((size_t)x % 16) == 0 && ((size_t)W % 16) == 0, "gemm_tc: x and W must be 16-byte aligned");
  GG_REQUIRE(mode >= 0 && mode <= 2, "gemm_tc: unknown mode %d", mode);
  GG_REQUIRE(mode != TC_OUT_SILU || N % 2 == 0, "gemm_tc: the gated product needs an even number of features");
  GG_REQUIRE(N % 2 == 0 || mode == TC_OUT_F32, "gemm_tc: bfloat16 rows of odd length are not 4-byte aligned");
  GG_REQUIRE(status != nullptr, "gemm_tc: no status word given");
  if (M == 0) return GG_OK;
  CUtensorMap map_x, map_w;
  int rc = gg_make_map_2d(&map_x, x, M, K, ldx, TC_BM);
  if (rc) return rc;
  const int w_rows = mode == TC_OUT_SILU ? 2 * N : N;
  rc = gg_make_map_2d(&map_w, W, w_rows, K, K, mode == TC_OUT_SILU ? 128 : 256);
  if (rc) return rc;
  const int n_tile = mode == TC_OUT_SILU ? 128 : 256;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + n_tile - 1) / n_tile;
  const long long num_tiles_ll = (long long)tiles_m * tiles_n;
  GG_REQUIRE(num_tiles_ll < (1ll << 30), "gemm_tc: too many tiles");
  const int num_tiles = (int)num_tiles_ll;
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  dim3 grid(num_tiles < num_sms ? num_tiles : num_sms);
  const size_t smem = (size_t)TC_STAGES * (TC_BM * TC_BK * 2 + 256 * TC_BK * 2) + 1024;
  cudaError_t e;
#define TC_LAUNCH(MODE)                                                                                   \
  do {                                                                                                    \
    static bool set = false;                                                                              \
    if (!set) {                                                                                           \
      e = cudaFuncSetAttribute(gemm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_tc: %s", cudaGetErrorString(e));            \
      set = true;                                                                                         \
    }                                                                                                     \
    e = gg_launch(gemm_tc_kernel<MODE>, grid, dim3(TC_THREADS), smem, stream, map_x, map_w, out, M, N, K, tiles_m, num_tiles, status, withhold_loads); \
  } while (0)
  if (mode == TC_OUT_BF16) TC_LAUNCH(TC_OUT_BF16);
  else if (mode == TC_OUT_F32) TC_LAUNCH(TC_OUT_F32);
  else TC_LAUNCH(TC_OUT_SILU);
#undef TC_LAUNCH
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_tc: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("gemm_tc");
}
