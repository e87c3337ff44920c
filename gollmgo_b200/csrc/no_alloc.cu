// gg_attn_decode_noalloc: split-KV decode attention whose scratch lives in a
// file-scope device array instead of caller-provided buffers.  See no_alloc.h for
// who needs it, the size limit and the rules of use.
#include "no_alloc.h"

#include <atomic>

#include "attention_common.cuh"

extern "C" int gg_attn_decode(const void* q, long long q_stride, const void* kcache,
                              const void* vcache, int dtype, const int* block_tables,
                              int bt_stride, const int* cu_q_lens, const int* context_lens,
                              const int* dec_seqs, int n_dec, int num_splits, float* part_o,
                              float* part_ml, void* out, int nh, int nkv, int d, int page_size,
                              int window, float scale, int allow_mma, cudaStream_t stream);

// The scratch itself.  In host code this name is only a stand-in for the symbol,
// not a device address: never hand it to a kernel.  The address comes from
// cudaGetSymbolAddress, below.
static __device__ __align__(256) float g_noalloc_scratch[GG_NOALLOC_MAX_PART_O + GG_NOALLOC_MAX_PART_ML];

#define GG_NOALLOC_MAX_DEVICES 64
// Per device, null until looked up.  Atomic, so two host threads that make their first call
// on a device at the same time both end up with the one address (each may look it up).
static std::atomic<float*> g_scratch_addr[GG_NOALLOC_MAX_DEVICES];

// Device address of the scratch array on the current device; looked up once per device.
static int scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= GG_NOALLOC_MAX_DEVICES)
    return gg_fail(GG_ERR_UNSUPPORTED, "attn_decode_noalloc: device index %d is beyond %d", dev, GG_NOALLOC_MAX_DEVICES);
  float* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return gg_fail(GG_ERR_CUDA, "attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *ptr = p;
  return GG_OK;
}

extern "C" int gg_attn_decode_noalloc(const void* q, long long q_stride, const void* kcache,
                                      const void* vcache, int dtype, const int* block_tables,
                                      int bt_stride, const int* cu_q_lens, const int* context_lens,
                                      const int* dec_seqs, int n_dec, int num_splits, void* out,
                                      int nh, int nkv, int d, int page_size, int window,
                                      float scale, int allow_mma, cudaStream_t stream) {
  // what is wrong with the arguments is said first, before the device is asked for anything
  GG_REQUIRE(n_dec >= 0 && num_splits >= 1 && num_splits <= 65535,
             "attn_decode_noalloc: bad n_dec %d or splits %d", n_dec, num_splits);
  GG_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_decode_noalloc: %d heads are not a multiple of %d kv heads", nh, nkv);
  GG_REQUIRE(d > 0 && d <= 256, "attn_decode_noalloc: head size %d is outside 1..256", d);
  GG_REQUIRE(page_size > 0 && bt_stride > 0, "attn_decode_noalloc: bad page size %d or block table width %d", page_size, bt_stride);
  const long long rows = (long long)n_dec * nh * num_splits;
  GG_REQUIRE(rows * d <= GG_NOALLOC_MAX_PART_O && rows * 2 <= GG_NOALLOC_MAX_PART_ML,
             "attn_decode_noalloc: %lld partial rows of %d floats exceed the built-in scratch "
             "(%d floats of outputs, %d of max/sum pairs): use fewer slices or gg_attn_decode "
             "with buffers of your own", rows, d, GG_NOALLOC_MAX_PART_O, GG_NOALLOC_MAX_PART_ML);
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  return gg_attn_decode(q, q_stride, kcache, vcache, dtype, block_tables, bt_stride, cu_q_lens,
                        context_lens, dec_seqs, n_dec, num_splits, scratch,
                        scratch + GG_NOALLOC_MAX_PART_O, out, nh, nkv, d, page_size, window, scale,
                        allow_mma, stream);
}
