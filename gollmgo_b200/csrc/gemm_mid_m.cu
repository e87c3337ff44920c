// Matrix products for a few dozen tokens (decode steps of 17 to 64 sequences, short prompt
// portions) on the fifth-generation tensor cores: out[M, N] = x[M, K] W[N, K]^T, bfloat16 in,
// float32 accumulation in tensor memory.
//
// With so few tokens the product is one pass over the weights, as in gemm_small_m.cu, but the
// tokens no longer fit one warp's registers.  Here the operands are swapped: rows of W are
// the M side of tcgen05.mma and the (padded) tokens its N side, so a CTA streams a slab of
// rows of W through shared memory once and the small x tile rides along.
//
// One pass over W is as fast as the SM with the most bytes, so the work is cut to the
// machine, not to the instruction: one CTA per SM with a deep ring, and the host chooses the
// slab's height (any number of rows up to 256: one or two TMA boxes of up to 128 rows, each
// the A operand of an M = 128 instruction whose unused rows are never read back) and the
// number S of CTAs that share a slab's K (a thread-block cluster) so that slabs x S comes as
// close to the SM count as whole clusters allow and every CTA takes in the same bytes.
//   warp 0  one lane issues the TMA loads per stage: the boxes of W (gate rows and the up rows
//           of the same features in the gated mode) and an NP x 64 tile of x.  The loads of
//           W for the first stages are issued before griddepcontrol.wait: the weights do not
//           depend on the kernel before this one, only x does.
//   warp 1  allocates tensor memory; one lane issues tcgen05.mma (M = 128, N = NP, K = 16)
//           and releases each stage with tcgen05.commit.
//   warps 2-5  read the accumulators with tcgen05.ld (thread = lane = row of a box).  S = 1:
//           epilogue and store straight from the registers.  S > 1: float32 [token][row] to
//           shared memory; after a cluster barrier every CTA sums its share of the rows over
//           all CTAs' partial results through distributed shared memory, in rank order (no
//           atomics), applies the epilogue and stores.
// Epilogues: bfloat16; float32; SiLU-gated: box 0 holds gate rows and box 1 the up rows of the
// same features (formula: kernels/gollmgo_ops.cu:361-374).
// Every wait on an mbarrier is bounded and reports through *status; the barriers of the
// cluster are reached by every thread whatever its waits returned.  No TMA load uses
// cluster multicast.
#include "tc_common.cuh"
#include <stdlib.h>

#define MM_BK 64
#define MM_THREADS 192
#define MM_BOX_BYTES (128 * MM_BK * 2)       // room of one box of W in a stage (128 rows, filled or not)
#define MM_RING_BYTES (220 * 1024)            // a CTA that has an SM to itself
#define MM_RING_BYTES_SHARED (108 * 1024)     // two CTAs on an SM
#define MM_MAX_STAGES 10

enum { MM_OUT_BF16 = 0, MM_OUT_F32 = 1, MM_OUT_SILU = 2 };
enum { MM_ERR_EMPTY_WAIT = 41, MM_ERR_FULL_WAIT = 42, MM_ERR_ACC_WAIT = 43, MM_ERR_DRAIN = 44 };

__host__ __device__ constexpr int mm_stage_bytes(int np, int boxes) { return boxes * MM_BOX_BYTES + np * MM_BK * 2; }
static int mm_stages(int np, int boxes, int per_sm) {
  const int n = (per_sm == 1 ? MM_RING_BYTES : MM_RING_BYTES_SHARED) / mm_stage_bytes(np, boxes);
  return n < MM_MAX_STAGES ? n : MM_MAX_STAGES;
}

__device__ __forceinline__ unsigned mm_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void mm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int MODE>
__device__ __forceinline__ void mm_store(void* out, size_t idx, float v) {
  if (MODE == MM_OUT_F32) reinterpret_cast<float*>(out)[idx] = v;
  else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// W floats at an address of the cluster's shared memory (from mapa).  No memory clobber: the
// loads of an output's partial results are in flight together; the barriers around the phase
// that uses them order them against the writes.
template <int W>
__device__ __forceinline__ void mm_ld_remote(float* v, unsigned addr) {
  if (W == 2) asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(addr));
  else asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[0]) : "r"(addr));
}

// The outputs of a slab that the CTA with this rank finishes: sums over the S partial results
// in rank order, epilogue, store.  W = 2: pairs of neighbouring outputs (box_rows, N and the
// address of out even enough).  Kept short on purpose: with six warps on an SM, what this
// phase costs is its instruction count.
template <int MODE, int BOXES, int W, int S>
__device__ __forceinline__ void mm_finish(void* out, unsigned dump_a, int M, int N, int n0, int box_rows, int rank) {
  constexpr bool GATED = MODE == MM_OUT_SILU;
  constexpr int DUMP_LD = BOXES * 128;
  unsigned base[S];                                   // this CTA's dump address in the shared memory of rank p
#pragma unroll
  for (int p = 0; p < S; ++p) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(base[p]) : "r"(dump_a), "r"(p));
  const int outs = GATED ? box_rows : BOXES * box_rows;
  const int groups = (outs + W - 1) / W;
  const int g_lo = rank * groups / S, per = (rank + 1) * groups / S - g_lo;
  if (per <= 0) return;
  int t = threadIdx.x / per, q = threadIdx.x - t * per;
  const int dt = MM_THREADS / per, dq = MM_THREADS - dt * per;
  while (t < M) {
    const int r = (g_lo + q) * W;
    const int col = (!GATED && BOXES == 2 && r >= box_rows) ? 128 + r - box_rows : r;
    const unsigned off = (unsigned)((t * DUMP_LD + col) * 4);
    float a[S][W], b[S][W];
#pragma unroll
    for (int p = 0; p < S; ++p) {
      mm_ld_remote<W>(a[p], base[p] + off);
      if (GATED) mm_ld_remote<W>(b[p], base[p] + off + 512);
    }
    float v[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float sa = a[0][w], sb = GATED ? b[0][w] : 0.f;
#pragma unroll
      for (int p = 1; p < S; ++p) { sa += a[p][w]; if (GATED) sb += b[p][w]; }
      v[w] = GATED ? __fdividef(sa, 1.f + __expf(-sa)) * sb : sa;
    }
    const int n = n0 + r;
    const size_t idx = (size_t)t * N + n;
    if (W == 2) {
      if (n < N) {                                    // n and N even: n + 1 < N as well
        if (MODE == MM_OUT_F32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + idx) = make_float2(v[0], v[W - 1]);
        else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(out) + idx) = __floats2bfloat162_rn(v[0], v[W - 1]);
      }
    } else if (n < N && r < outs) {
      mm_store<MODE>(out, idx, v[0]);
    }
    q += dq;
    t += dt;
    if (q >= per) { q -= per; ++t; }
  }
}
template <int MODE, int BOXES, int W>
__device__ __forceinline__ void mm_finish_any(void* out, unsigned dump_a, int M, int N, int n0, int box_rows, int S, int rank) {
  if (S == 1) mm_finish<MODE, BOXES, W, 1>(out, dump_a, M, N, n0, box_rows, rank);
  else if (S == 2) mm_finish<MODE, BOXES, W, 2>(out, dump_a, M, N, n0, box_rows, rank);
  else if (S == 4) mm_finish<MODE, BOXES, W, 4>(out, dump_a, M, N, n0, box_rows, rank);
  else mm_finish<MODE, BOXES, W, 8>(out, dump_a, M, N, n0, box_rows, rank);
}

// grid (S, slabs), cluster (S, 1, 1): CTA (s, t) multiplies slab t over its share of K.
// BOXES boxes of box_rows rows of W per slab (the gated mode: box 0 gate rows, box 1 up rows).
template <int MODE, int NP, int BOXES>
__global__ void __launch_bounds__(MM_THREADS, 1)
gemm_mid_m_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  void* __restrict__ out, int M, int N, int K, int box_rows, int pairs, int stages,
                  int* __restrict__ status) {
  constexpr unsigned X_BYTES = NP * MM_BK * 2, W_BYTES = BOXES * MM_BOX_BYTES, STAGE_BYTES = W_BYTES + X_BYTES;
  const int STAGES = stages;
  constexpr unsigned TMEM_COLS = BOXES * NP;                             // 32, 64 or 128: a power of two
  constexpr int DUMP_LD = BOXES * 128;
  extern __shared__ unsigned char mm_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * MM_MAX_STAGES + 1];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned tiles = (tc_smem(mm_smem_raw) + 1023u) & ~1023u;        // 1024-byte aligned stages
  unsigned char* tiles_ptr = mm_smem_raw + (tiles - tc_smem(mm_smem_raw));
  const unsigned full0 = tc_smem(&bars[0]), empty0 = tc_smem(&bars[MM_MAX_STAGES]), acc_full = tc_smem(&bars[2 * MM_MAX_STAGES]);
  const int S = gridDim.x, rank = (int)mm_cluster_rank();
  const int slab = blockIdx.y;
  const int num_kb = (K + MM_BK - 1) / MM_BK;
  const int kb0 = (int)((long long)rank * num_kb / S), kb1 = (int)((long long)(rank + 1) * num_kb / S);
  const int my_kb = kb1 - kb0;
  // first output of the slab: box_rows gated features, or BOXES * box_rows rows of W
  const int n0 = MODE == MM_OUT_SILU ? slab * box_rows : slab * BOXES * box_rows;
  const unsigned tx_bytes = (unsigned)(BOXES * box_rows * MM_BK * 2) + X_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(acc_full, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
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
      const int s = i % STAGES;
      const unsigned dst = tiles + s * STAGE_BYTES, bar = full0 + 8 * s;
      const int k = (kb0 + i) * MM_BK;
      tma_load_2d(dst, &map_w, k, n0, bar);
      if (BOXES == 2) tma_load_2d(dst + MM_BOX_BYTES, &map_w, k, MODE == MM_OUT_SILU ? N + n0 : n0 + box_rows, bar);
    };
    auto load_x = [&](int i) {
      const int s = i % STAGES;
      tma_load_2d(tiles + s * STAGE_BYTES + W_BYTES, &map_x, (kb0 + i) * MM_BK, 0, full0 + 8 * s);
    };
    // the weights of the first stages, before the kernel ahead has finished; then its output
    const int early = min(STAGES, my_kb);
    for (int i = 0; i < early; ++i) { mbar_expect_tx(full0 + 8 * i, tx_bytes); load_w(i); }
    pdl_wait();
    for (int i = 0; i < early; ++i) load_x(i);
    int issued = early;
    for (int i = early; i < my_kb; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1)) { atomicExch(status, MM_ERR_EMPTY_WAIT); atomicExch(&abort_s, 1); break; }
      if (*(volatile int*)&abort_s) break;
      mbar_expect_tx(full0 + 8 * s, tx_bytes);
      load_w(i);
      load_x(i);
      issued = i + 1;
    }
    // on an abort: let the copies that were issued land before shared memory is reused
    if (*(volatile int*)&abort_s) {
      for (int i = max(0, issued - STAGES); i < issued; ++i)
        if (!mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1)) { atomicExch(status, MM_ERR_DRAIN); break; }
    }
  } else {
    pdl_wait();
    if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer: A = a box of W (M = 128), B = the tokens (N = NP), both K-major
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NP >> 3) << 17) | ((128u >> 4) << 24);
      for (int i = 0; i < my_kb; ++i) {
        const int s = i % STAGES;
        if (*(volatile int*)&abort_s) break;
        if (!mbar_wait(full0 + 8 * s, (i / STAGES) & 1)) { atomicExch(status, MM_ERR_FULL_WAIT); atomicExch(&abort_s, 1); break; }
        tc_fence_after();
        const unsigned long long a_desc = tc_smem_desc(tiles + s * STAGE_BYTES);
        const unsigned long long a1_desc = tc_smem_desc(tiles + s * STAGE_BYTES + MM_BOX_BYTES);
        const unsigned long long b_desc = tc_smem_desc(tiles + s * STAGE_BYTES + W_BYTES);
#pragma unroll
        for (int k = 0; k < MM_BK / 16; ++k) {
          const unsigned acc = (i > 0 || k > 0) ? 1u : 0u;
          tc_mma(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, acc);
          if (BOXES == 2) tc_mma(tmem_base + NP, a1_desc + 2 * k, b_desc + 2 * k, idesc, acc);
        }
        tc_commit(empty0 + 8 * s);
      }
      tc_commit(acc_full);                           // the accumulators are complete (also on abort)
    }
  }
  // ---------------- accumulators -> shared memory as float32 [token][box][row], over the stages
  float* dump = reinterpret_cast<float*>(tiles_ptr);                     // [NP][BOXES * 128]
  if (warp >= 2) {
    const int quarter = warp & 3, row = quarter * 32 + lane;
    bool ok = mbar_wait(acc_full, 0);
    if (!ok) { atomicExch(status, MM_ERR_ACC_WAIT); atomicExch(&abort_s, 1); }
    ok = __all_sync(0xffffffffu, ok && !*(volatile int*)&abort_s);
    tc_fence_after();
    const unsigned acc = tmem_base + ((unsigned)(quarter * 32) << 16);
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < NP && c < M; c += 32) {
        unsigned va[32], vb[32];
        if (my_kb > 0) {
          tc_load32(acc + c, va);
          if (BOXES == 2) tc_load32(acc + NP + c, vb);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) { va[j] = 0u; vb[j] = 0u; }     // no share of K: nothing was accumulated
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          dump[(c + j) * DUMP_LD + row] = __uint_as_float(va[j]);
          if (BOXES == 2) dump[(c + j) * DUMP_LD + 128 + row] = __uint_as_float(vb[j]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (S > 1) mm_cluster_sync();                      // every CTA's partial result is in its shared memory
  // ---------------- this CTA's share of the slab's outputs, summed over the cluster in rank order
  if (!*(volatile int*)&abort_s) {
    const unsigned dump_a = tc_smem(dump);
    // two neighbouring outputs per thread where rows of out keep pairs aligned, else one
    if (pairs) mm_finish_any<MODE, BOXES, 2>(out, dump_a, M, N, n0, box_rows, S, rank);
    else mm_finish_any<MODE, BOXES, 1>(out, dump_a, M, N, n0, box_rows, S, rank);
  }
  if (S > 1) mm_cluster_sync();                      // nobody leaves while a neighbour may still read it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
template <typename Kern>
static cudaError_t mm_launch(Kern kernel, dim3 grid, size_t smem, int cluster_x, cudaStream_t stream,
                             const CUtensorMap& map_x, const CUtensorMap& map_w, void* out, int M, int N, int K,
                             int box_rows, int pairs, int stages, int* status) {
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
  return cudaLaunchKernelEx(&cfg, kernel, map_x, map_w, out, M, N, K, box_rows, pairs, stages, status);
}

static size_t mm_smem_bytes(int np, int boxes, int per_sm) {
  return (size_t)mm_stages(np, boxes, per_sm) * mm_stage_bytes(np, boxes) + 1024;
}

// Clusters of S CTAs of this kernel, one CTA on an SM, that the device holds at once (all
// variants take the same shared memory within a few KB, so one answers for all).  0 if the
// device takes no such cluster.
static int mm_cluster_places(int S) {
  static int cached[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (cached[S] >= 0) return cached[S];
  auto kernel = gemm_mid_m_kernel<MM_OUT_BF16, 64, 1>;
  const size_t smem = mm_smem_bytes(64, 1, 1);
  int n = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_RING_BYTES + 1024) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, 1024);
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
  } else {
    (void)cudaGetLastError();
  }
  return cached[S] = n;
}

static int mm_env_int(const char* name) { const char* v = getenv(name); return v ? atoi(v) : 0; }
struct MmPlan { int S, boxes, box_rows, slabs, per_sm, at_once; };

// How a product of `rows` rows of W (gated: features) is cut.
//   Many rows (the gated product, any matrix with at least 64 rows per SM): one CTA on an SM
//   with a deep ring, slabs as high as it takes for slabs x S to fill whole rounds of the
//   places that clusters of S have (places_of(S)); S chosen to make the bytes the busiest CTA
//   takes in least (W and the x tile that comes with every K block), with a charge for the
//   merge through the cluster.  The gated product of the Llama-3.1-8B shape: 147 slabs of 98
//   features, S = 1, 43 us at 64 tokens against 48 with 224 slabs of 64 on 296 places.
//   Few rows (qkv, o, down): slabs of 128 rows, two CTAs on an SM with half the ring each, K
//   split over as many CTAs as still fit the machine at once; measured better than one CTA per
//   SM for these (o: 13.0 against 14.4 us, down: 25.9 against 28.4), whose time is start,
//   merge and end more than bytes, which two CTAs on an SM overlap.
template <typename Places>
static MmPlan mm_plan(int rows, int num_kb, int np, bool gated, int num_sms, Places places_of, int force_S, int force_per_sm) {
  const bool deep = force_per_sm ? force_per_sm == 1 : (gated || rows >= 64 * num_sms);
  if (!deep) {
    MmPlan p = {1, 1, 128, (rows + 127) / 128, 2, 2 * num_sms};
    while (p.S < 8 && p.slabs * (p.S * 2) <= 2 * num_sms && p.S * 2 <= num_kb) p.S *= 2;
    if (force_S && force_S <= num_kb) p.S = force_S;
    return p;
  }
  const int cap = gated ? 128 : 256;
  MmPlan best = {0, 0, 0, 0, 1, 0};
  double best_cost = -1;
  for (int S = 1; S <= 8 && S <= num_kb; S *= 2) {
    if (force_S && S != force_S) continue;
    const int places = places_of(S);
    if (places < 1) continue;
    int R = (rows + places - 1) / places;
    if (R < 16) R = rows < 16 ? rows : 16;
    if (R > cap) R = cap;
    if (R % 2 && R < cap && rows > 1) ++R;             // even, so that pairs of outputs stay aligned
    MmPlan p = {S, 1, R, 0, 1, places * S};
    if (gated) { p.boxes = 2; p.box_rows = R; }
    else if (R > 128) { p.boxes = 2; p.box_rows = ((R + 3) / 4) * 2; }
    const int slab_rows = gated ? p.box_rows : p.boxes * p.box_rows;
    p.slabs = (rows + slab_rows - 1) / slab_rows;
    const int rounds = (p.slabs + places - 1) / places;
    const double stage = (double)p.boxes * p.box_rows * 128 + np * 128.0;
    const double cost = stage * ((num_kb + S - 1) / S) * rounds + (S > 1 ? 40960.0 * S : 0.0);
    if (best_cost < 0 || cost < best_cost) { best = p; best_cost = cost; }
  }
  if (best.S == 0) {                                 // a forced S that the device or K does not take
    const int R = rows < 128 ? (rows + (rows > 1 ? rows % 2 : 0)) : 128;
    best = MmPlan{1, gated ? 2 : 1, R, (rows + R - 1) / R, 1, num_sms};
  }
  return best;
}

// The plan for a shape on this device: plan[0..5] = S, boxes, box_rows, slabs, CTAs per SM,
// CTAs that run at once.  GOLLMGO_B200_GEMM_MID_SPLIT (1, 2, 4, 8) and
// GOLLMGO_B200_GEMM_MID_PER_SM (1, 2) force a choice, for measurements.
extern "C" int gg_gemm_mid_m_plan(int M, int N, int K, int mode, int* plan) {
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
      num_sms = 148;
  }
  static const int force_S = mm_env_int("GOLLMGO_B200_GEMM_MID_SPLIT"), force_per_sm = mm_env_int("GOLLMGO_B200_GEMM_MID_PER_SM");
  const int np = M <= 32 ? 32 : 64, num_kb = (K + MM_BK - 1) / MM_BK;
  auto places_of = [&](int S) {
    const int fit = num_sms / S;
    if (S == 1) return fit;
    const int clusters = mm_cluster_places(S);
    return clusters < fit ? clusters : fit;
  };
  const MmPlan p = mm_plan(N, num_kb, np, mode == MM_OUT_SILU, num_sms, places_of,
                           force_S == 1 || force_S == 2 || force_S == 4 || force_S == 8 ? force_S : 0,
                           force_per_sm == 1 || force_per_sm == 2 ? force_per_sm : 0);
  if (plan) { plan[0] = p.S; plan[1] = p.boxes; plan[2] = p.box_rows; plan[3] = p.slabs; plan[4] = p.per_sm; plan[5] = p.at_once; }
  return GG_OK;
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
  int plan[6];
  gg_gemm_mid_m_plan(M, N, K, mode, plan);
  const int S = plan[0], boxes = plan[1], box_rows = plan[2], slabs = plan[3], per_sm = plan[4];
  GG_REQUIRE(slabs <= 65535, "gemm_mid_m: too many row slabs (%d)", slabs);
  CUtensorMap map_x, map_w;
  int rc = gg_make_map_2d(&map_x, x, M, K, ldx, np);
  if (rc) return rc;
  rc = gg_make_map_2d(&map_w, W, mode == MM_OUT_SILU ? 2 * N : N, K, K, box_rows);
  if (rc) return rc;
  const int stages = mm_stages(np, boxes, per_sm);
  const size_t smem = mm_smem_bytes(np, boxes, per_sm);
  const int pairs = box_rows % 2 == 0 && N % 2 == 0 && ((size_t)out % 8) == 0;
  dim3 grid(S, slabs);
  cudaError_t e = cudaSuccess;
#define MM_LAUNCH(MODE, NP, BOXES)                                                                         \
  do {                                                                                                     \
    static bool set = false;                                                                               \
    if (!set) {                                                                                            \
      e = cudaFuncSetAttribute(gemm_mid_m_kernel<MODE, NP, BOXES>, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_RING_BYTES + 1024); \
      if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_mid_m: %s", cudaGetErrorString(e));          \
      set = true;                                                                                          \
    }                                                                                                      \
    e = mm_launch(gemm_mid_m_kernel<MODE, NP, BOXES>, grid, smem, S, stream, map_x, map_w, out, M, N, K, box_rows, pairs, stages, status); \
  } while (0)
#define MM_LAUNCH_NP(MODE, BOXES) do { if (np == 32) MM_LAUNCH(MODE, 32, BOXES); else MM_LAUNCH(MODE, 64, BOXES); } while (0)
  if (mode == MM_OUT_SILU) MM_LAUNCH_NP(MM_OUT_SILU, 2);
  else if (mode == MM_OUT_F32) { if (boxes == 2) MM_LAUNCH_NP(MM_OUT_F32, 2); else MM_LAUNCH_NP(MM_OUT_F32, 1); }
  else { if (boxes == 2) MM_LAUNCH_NP(MM_OUT_BF16, 2); else MM_LAUNCH_NP(MM_OUT_BF16, 1); }
#undef MM_LAUNCH_NP
#undef MM_LAUNCH
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "gemm_mid_m: launch: %s", cudaGetErrorString(e));
  return gg_check_launch("gemm_mid_m");
}
