"""The native packing of decode steps (csrc/host_pack.cu) against the general path of
BatchBuilder.build: the same device arrays for the same requests, over many steps that cross
page borders, with a windowed group beside a full one, padding to a fixed layout, requests
that end and slots that are used again."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def run(native: bool, seed: int, fixed: bool):
    from gollmgo_b200.cache import CacheManager, PagedKVNeed
    from gollmgo_b200.engine.batch import BatchBuilder, StepEntry
    rng = random.Random(seed)
    needs = [PagedKVNeed(2, 16, None), PagedKVNeed(2, 16, 20), PagedKVNeed(2, 16, None)]   # two groups
    cm = CacheManager(needs, 8, 64, 6, dtype=torch.bfloat16, device="cuda")
    from gollmgo_b200.parts import QueryTiles
    bb = BatchBuilder(cm, "cuda", query_tiles=[QueryTiles(16), QueryTiles(32, most_keys_first=True)])
    bb.native_decode = native
    static = torch.zeros(4096, dtype=torch.int32, device="cuda") if fixed else None
    live, out, next_id = [], [], 0
    for step in range(120):
        while len(live) < 5 and rng.random() < 0.5:
            rid = f"r{next_id}"
            next_id += 1
            cm.admit(rid)
            n = rng.randint(1, 19)
            bb.build([StepEntry(rid, list(range(n)), [])])          # a prompt portion: the general path
            live.append(rid)
        if not live:
            continue
        chosen = [r for r in live if rng.random() < 0.8] or live[:1]
        entries = [StepEntry(r, [rng.randrange(100)], [0], token_src=(i if rng.random() < 0.5 else -1))
                   for i, r in enumerate(chosen)]
        sb = bb.build(entries, fixed_seqs=6 if fixed else None, fixed_stride=16 if fixed else None,
                      static_dev=static)
        torch.cuda.synchronize()
        B = sb.num_seqs
        rec = {"tokens": sb.token_ids[:B].tolist(), "pos": sb.positions[:B].tolist(),
               "src": None if sb.token_src is None else sb.token_src[:B].tolist(),
               "cu": sb.cu_q_lens.tolist(), "ctx": sb.context_lens[:B].tolist(),
               "slots": sb.state_slots[:B].tolist(), "rows": sb.logit_rows.tolist(), "dec": sb.dec_seqs.tolist(),
               "sm": [s[:B].tolist() for s in sb.slot_mapping],
               "bt": [t.view(B, sb.bt_stride).tolist() for t in sb.block_tables],
               "facts": (sb.num_tokens, sb.num_seqs, sb.num_logit_rows, sb.num_portions, sb.num_decode, sb.bt_stride,
                         sb.request_ids, sb.q_lens, sb.q_starts, sb.state_slot_list)}
        if fixed:
            # columns beyond the ones in use keep what an earlier step left there; compare what a kernel may read
            for g, t in enumerate(rec["bt"]):
                for b, row in enumerate(t):
                    n = -(-rec["ctx"][b] // 8) if b < len(chosen) else 0
                    t[b] = row[:n]
        out.append(rec)
        for r in list(chosen):
            if rng.random() < 0.07:
                cm.free(r)
                live.remove(r)
        cm.audit()
    return out


@pytest.mark.parametrize("fixed", [False, True])
def test_native_decode_packing_equals_the_general_path(cuda_device, fixed):
    a, b = run(True, 5, fixed), run(False, 5, fixed)
    assert len(a) == len(b) and len(a) > 50
    for i, (x, y) in enumerate(zip(a, b)):
        assert x == y, f"step {i}"


def test_native_decode_packing_is_all_or_nothing(cuda_device):
    from gollmgo_b200.cache import CacheManager, OutOfPages, PagedKVNeed
    from gollmgo_b200.engine.batch import BatchBuilder, StepEntry
    cm = CacheManager([PagedKVNeed(1, 16, None)], 8, 3, 4, dtype=torch.bfloat16, device="cuda")
    bb = BatchBuilder(cm, "cuda")
    for r, n in (("a", 8), ("b", 8), ("c", 7)):
        cm.admit(r)
        bb.build([StepEntry(r, [0] * n, [])])
    assert cm.free_pages() == 0
    with pytest.raises(OutOfPages):                       # c fits, a needs a page that is not there
        bb.build([StepEntry("c", [1], [0]), StepEntry("a", [1], [0])])
    assert cm.num_tokens("c") == 7 and cm.num_tokens("a") == 8
    cm.audit()
