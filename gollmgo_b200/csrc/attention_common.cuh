// Argument block shared by the attention kernels, and the tensor-core helpers of
// the bfloat16 fast path (mma.sync m16n8k16, ldmatrix, cp.async, shared-memory swizzle).
#pragma once
#include "common.cuh"

struct AttnArgs {
  const void* q;            // [T, q_stride]: head h of token t at q + t*q_stride + h*d
  long long q_stride;
  const void* kcache;       // [num_pages, nkv, page_size, d]
  const void* vcache;
  const int* block_tables;  // [B, bt_stride]; -1 = page given back (behind the window)
  int bt_stride;
  const int* cu_q_lens;     // [B+1]
  const int* context_lens;  // [B] tokens in the cache after this step's write
  void* out;                // [T, nh*d]
  int nh, nkv, d, page_size, window;
  float scale;
  // prompt portions
  const int* tile_seq;      // [num_tiles]
  const int* tile_q0;       // [num_tiles] offset of the tile in the sequence's portion
  // decoded tokens
  const int* dec_seqs;      // [n_dec] sequence indices with exactly one query token; -1 = padding
  int num_splits;
  float* part_o;            // [n_dec, nh, num_splits, d]
  float* part_ml;           // [n_dec, nh, num_splits, 2]
  // decode with the rotation fused in (attention_mma.cu): q is then the raw [T, (nh+2nkv)*d]
  // projection output, and the kernel rotates q and k itself and writes k and v to the cache
  const double* rope_inv_freq;   // d/2 inverse frequencies, or null: q and the cache are ready
  const int* rope_positions;     // [T]
  const int* slot_mapping;       // [T] page * page_size + offset, < 0: no write
  int rope_write_cache;
};

// General kernels (attention.cu)
int attn_prefill_general(const AttnArgs& a, int dtype, int num_tiles, cudaStream_t stream);
int attn_decode_general(const AttnArgs& a, int dtype, int n_dec, cudaStream_t stream);
int attn_merge_launch(const AttnArgs& a, int dtype, int n_dec, cudaStream_t stream);
// bfloat16 tensor-core kernels for head sizes 64 and 128 (attention_mma.cu)
bool attn_mma_supported(int dtype, int d);
int attn_prefill_mma(const AttnArgs& a, int num_tiles, cudaStream_t stream);   // tiles of 64 queries
#define ATTN_MAX_CLUSTER 8       // slices of one token and kv head that can be one (portable) cluster
int attn_decode_mma(const AttnArgs& a, int n_dec, cudaStream_t stream, bool* merged);
int attn_decode_cluster_capacity(int d, int splits, int group);
// large batches: the tiles of all (token, kv head) pairs cut into equal ranges, one per CTA
int attn_decode_flat_ctas(int d);
int attn_decode_flat(const AttnArgs& a, int n_dec, int* prefix, cudaStream_t stream);
// bfloat16 tcgen05 kernel for prompt portions, head size 128 (attention_tc.cu); tiles of 128 queries
bool attn_tc_supported(int dtype, int d, int page_size);
int attn_prefill_tc(const AttnArgs& a, int num_tiles, int T, int num_pages, int* status, cudaStream_t stream);
// the same with two heads of one kv head per CTA (attention_tc2.cu): even groups of heads, pages of up to 64 tokens
bool attn_tc2_supported(int dtype, int d, int page_size, int nh, int nkv);
int attn_prefill_tc2(const AttnArgs& a, int num_tiles, int T, int num_pages, int* status, cudaStream_t stream);
// the same in steps of 128 keys (attention_tc3.cu)
bool attn_tc3_supported(int dtype, int d, int page_size, int nh, int nkv);
int attn_prefill_tc3(const AttnArgs& a, int num_tiles, int T, int num_pages, int* status, cudaStream_t stream);

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
