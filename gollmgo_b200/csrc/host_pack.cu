// Host side of a decode step: packs the int32 buffer that one copy sends to the device
// (token ids, positions, slots of the new keys, lengths, block tables, ...) for a step in
// which every sequence brings exactly one token and wants its logits.  This is the loop
// that runs once per generated token of every request, so it is native code over flat
// arrays: the cache manager keeps, per group of layers, a table [state slot][logical page]
// of page ids (-1 = none) and the engine hands over the step's state slots, token ids and
// context lengths.  The reference builds the same facts in Go each step
// (internal/scheduler/fcfs.go:64-200, internal/backend/cuda/model_bridge.go:305-383).
// No device code here.
#include "common.cuh"

// off: offsets (in ints) into h of token_ids, token_src, positions, cu_q_lens, context_lens,
// state_slots, logit_rows, dec_seqs, then G slot_mapping arrays, then G block tables.
// B real sequences, padded to Bp (padding: token 0, no source, no slot, no pages; its logits
// row is computed and ignored).  used = columns of the packed block tables.
extern "C" int gg_pack_decode_step(int* h, const int* off, int G, int B, int Bp, int used, int page_size,
                                   const int* tokens, const int* token_src, const int* state_slots,
                                   const int* context_after, const int* const* tables, const int* table_width) {
  GG_REQUIRE(h && off && tokens && token_src && state_slots && context_after && tables && table_width,
             "pack_decode_step: a null argument");
  GG_REQUIRE(G >= 0 && B >= 1 && Bp >= B && used >= 1 && page_size > 0 && (page_size & (page_size - 1)) == 0,
             "pack_decode_step: bad sizes G=%d B=%d Bp=%d used=%d page=%d", G, B, Bp, used, page_size);
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  const int mask = page_size - 1;
  int* tok = h + off[0];
  int* src = h + off[1];
  int* pos = h + off[2];
  int* cu = h + off[3];
  int* ctx = h + off[4];
  int* st = h + off[5];
  int* rows = h + off[6];
  int* dec = h + off[7];
  for (int b = 0; b < Bp; ++b) {
    const bool real = b < B;
    tok[b] = real ? tokens[b] : 0;
    src[b] = real ? token_src[b] : -1;
    pos[b] = real ? context_after[b] - 1 : 0;
    cu[b] = b;
    ctx[b] = real ? context_after[b] : 0;
    st[b] = real ? state_slots[b] : -1;
    rows[b] = b;
    dec[b] = real ? b : -1;
  }
  cu[Bp] = Bp;
  for (int g = 0; g < G; ++g) {
    int* sm = h + off[8 + g];
    int* bt = h + off[8 + G + g];
    const int* tab = tables[g];
    const int width = table_width[g];
    for (int b = 0; b < Bp; ++b) {
      int* row = bt + (size_t)b * used;
      if (b >= B) {
        sm[b] = -1;
        for (int c = 0; c < used; ++c) row[c] = -1;
        continue;
      }
      const int* src_row = tab + (size_t)state_slots[b] * width;
      const int p = context_after[b] - 1, lp = p >> shift;
      GG_REQUIRE(lp < width && src_row[lp] >= 0, "pack_decode_step: sequence %d has no page for position %d", b, p);
      sm[b] = src_row[lp] * page_size + (p & mask);
      const int n = used < width ? used : width;
      for (int c = 0; c < n; ++c) row[c] = src_row[c];
      for (int c = n; c < used; ++c) row[c] = -1;
    }
  }
  return GG_OK;
}
