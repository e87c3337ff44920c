"""The reference arm of bench.py: TensorGreed/gollmgo's own engine below its Go host.

gollmgo is a Go program; everything it runs on the GPU sits behind a C API in five CUDA
files (kernels/gollmgo_backend.cu, gollmgo_ops.cu, gollmgo_model.cu, gollmgo_paged_attn.cu,
gollmgo_kvcache.cu) that its Makefile builds with nvcc alone (Makefile:49-73).  This module
compiles those five files UNMODIFIED into ``baseline/_ref/libgollmgo_ref.so`` and drives the
C API with ctypes the way the Go bridge does (internal/backend/cuda/model_bridge.go:207-290):
``gollmgo_model_create`` / ``_load_weight`` / ``_ready`` (kernels/gollmgo_model.cu:306-548),
``gollmgo_kvcache_create`` (kernels/gollmgo_kvcache.cu:23-63), one
``gollmgo_model_forward_prefill`` call per prompt (:901-952) and one
``gollmgo_model_forward_paged`` call per decode step (:954-1063), with the next tokens chosen
on the host from the logits it returns, as its engine does (internal/engine/sampling.go:75-85).

Nothing of gollmgo_b200 is imported here: no model, kernel, cache or engine of this
repository is on this path.  Only numpy and ctypes are used; the CUDA runtime and cuBLAS are
the ones the reference links against.
"""
from __future__ import annotations

import ctypes
import json
import os
import shutil
import subprocess
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(REF_DIR, "libgollmgo_ref.so")
KERNEL_FILES = ["gollmgo_backend.cu", "gollmgo_ops.cu", "gollmgo_model.cu", "gollmgo_paged_attn.cu",
                "gollmgo_kvcache.cu"]
GOLLMGO_DTYPE_BF16 = 1               # kernels/gollmgo_model.h:22


class Unavailable(RuntimeError):
    """The reference cannot be built or refuses to run here; the message is the reason."""


def _source_dir() -> str:
    for d in (os.environ.get("GOLLMGO_REFERENCE_KERNELS"), "/root/reference/kernels",
              os.path.join(REF_DIR, "kernels")):
        if d and all(os.path.exists(os.path.join(d, f)) for f in KERNEL_FILES):
            return d
    raise Unavailable("the reference's kernels/*.cu are not on this machine and no built "
                      "baseline/_ref/libgollmgo_ref.so came with the repository")


def build(verbose: bool = False) -> str:
    """Compile the reference's five CUDA files, as they are, into one shared object."""
    if os.path.exists(LIB):
        return LIB
    src = _source_dir()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise Unavailable("nvcc not found: cannot build the reference's kernels")
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = [nvcc, "-arch=sm_100", "-O2", "-shared", "-Xcompiler", "-fPIC", "-o", LIB + ".tmp",
           *[os.path.join(src, f) for f in KERNEL_FILES], "-lcublas", "-lcudart"]
    if verbose:
        print("[reference] " + " ".join(cmd), file=sys.stderr, flush=True)
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise Unavailable("nvcc failed on the reference's kernels: " + (p.stderr or p.stdout).strip()[-300:])
    os.replace(LIB + ".tmp", LIB)
    return LIB


class ModelConfig(ctypes.Structure):
    """gollmgo_model_config_t (kernels/gollmgo_model.h:28-40)."""
    _fields_ = [("num_layers", ctypes.c_int), ("hidden_size", ctypes.c_int),
                ("intermediate_size", ctypes.c_int), ("num_heads", ctypes.c_int),
                ("num_kv_heads", ctypes.c_int), ("vocab_size", ctypes.c_int),
                ("max_seq_len", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("rms_norm_eps", ctypes.c_float), ("dtype", ctypes.c_int), ("quant_dtype", ctypes.c_int)]


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class Reference:
    """One model + KV cache of the reference, through its C API."""

    def __init__(self, cfg: dict, max_seq_len: int, num_slots: int, device: int = 0):
        lib = ctypes.CDLL(build())
        self.lib = lib
        self.rt = ctypes.CDLL("libcudart.so.12")
        vp = ctypes.c_void_p
        lib.gollmgo_backend_create.argtypes = [ctypes.c_int, ctypes.POINTER(vp)]
        lib.gollmgo_model_create.argtypes = [vp, ctypes.POINTER(ModelConfig), ctypes.POINTER(vp)]
        lib.gollmgo_model_load_weight.argtypes = [vp, ctypes.c_char_p, vp, ctypes.c_int64, ctypes.c_char_p]
        lib.gollmgo_model_ready.argtypes = [vp]
        lib.gollmgo_kvcache_create.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.POINTER(vp)]
        ip, fp = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float)
        lib.gollmgo_model_forward.argtypes = [vp, vp, ip, ip, ctypes.c_int, fp]
        lib.gollmgo_model_forward_prefill.argtypes = [vp, vp, ip, ip, ip, ctypes.c_int, vp, fp]
        lib.gollmgo_model_forward_paged.argtypes = [vp, vp, ip, ip, ip, ctypes.c_int, vp, ip, ip,
                                                    ctypes.c_int, ctypes.c_int, ip, fp]
        lib.gollmgo_model_destroy.argtypes = [vp]
        lib.gollmgo_kvcache_destroy.argtypes = [vp]
        lib.gollmgo_backend_destroy.argtypes = [vp]
        lib.gollmgo_backend_last_error.argtypes = [vp]
        lib.gollmgo_backend_last_error.restype = ctypes.c_char_p
        self.cfg = cfg
        self.V = cfg["vocab_size"]
        self.backend, self.model, self.kv = vp(), vp(), vp()
        self._ok(lib.gollmgo_backend_create(device, ctypes.byref(self.backend)), "gollmgo_backend_create")
        nh = cfg["num_attention_heads"]
        mc = ModelConfig(cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], nh,
                         cfg.get("num_key_value_heads") or nh, self.V, max_seq_len,
                         cfg.get("head_dim") or cfg["hidden_size"] // nh,
                         float(cfg.get("rms_norm_eps", 1e-5)), GOLLMGO_DTYPE_BF16, 0)
        self.mc = mc
        self._ok(lib.gollmgo_model_create(self.backend, ctypes.byref(mc), ctypes.byref(self.model)),
                 "gollmgo_model_create")
        self.num_slots = num_slots
        self.max_seq_len = max_seq_len
        self._kv_made = False

    def _ok(self, status: int, what: str) -> None:
        if status != 0:
            raise Unavailable(f"the reference's {what} returned status {status}")

    def load(self, name: str, bits: np.ndarray) -> None:
        """Hand one tensor (bfloat16 bit patterns) to gollmgo_model_load_weight."""
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        self._ok(self.lib.gollmgo_model_load_weight(self.model, name.encode(), bits.ctypes.data,
                                                    bits.nbytes, b"BF16"), f"gollmgo_model_load_weight({name})")

    def ready(self) -> None:
        self._ok(self.lib.gollmgo_model_ready(self.model), "gollmgo_model_ready")
        mc = self.mc
        self._ok(self.lib.gollmgo_kvcache_create(self.backend, mc.num_layers, self.num_slots, mc.num_kv_heads,
                                                 mc.head_dim, ctypes.byref(self.kv)), "gollmgo_kvcache_create")
        self._kv_made = True

    # ------------------------------------------------------------------ the three forward calls
    def forward(self, tokens, positions, out: np.ndarray) -> None:
        t, tp = _i32(tokens)
        p, pp = _i32(positions)
        self._ok(self.lib.gollmgo_model_forward(self.backend, self.model, tp, pp, len(t),
                                                out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))),
                 "gollmgo_model_forward")

    def prefill(self, tokens, positions, slots, out: np.ndarray) -> None:
        t, tp = _i32(tokens)
        p, pp = _i32(positions)
        s, sp = _i32(slots)
        self._ok(self.lib.gollmgo_model_forward_prefill(self.backend, self.model, tp, pp, sp, len(t), self.kv,
                                                        out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))),
                 "gollmgo_model_forward_prefill")

    def decode(self, tokens, positions, slots, seq_lens, slot_tables: np.ndarray, out: np.ndarray) -> None:
        """One decode step of len(tokens) sequences; slot_tables is [n, max context] as the Go
        bridge pads it (model_bridge.go:262-276)."""
        t, tp = _i32(tokens)
        p, pp = _i32(positions)
        s, sp = _i32(slots)
        l, lp = _i32(seq_lens)
        st, stp = _i32(slot_tables)
        n = len(t)
        counts, cp = _i32(np.ones(n))
        self._ok(self.lib.gollmgo_model_forward_paged(self.backend, self.model, tp, pp, sp, n, self.kv, lp, stp,
                                                      n, st.shape[1], cp,
                                                      out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))),
                 "gollmgo_model_forward_paged")

    def close(self) -> None:
        if self._kv_made:
            self.lib.gollmgo_kvcache_destroy(self.kv)
        self.lib.gollmgo_model_destroy(self.model)
        self.lib.gollmgo_backend_destroy(self.backend)

    # ------------------------------------------------------------------ device timing
    def event(self):
        e = ctypes.c_void_p()
        if self.rt.cudaEventCreate(ctypes.byref(e)) != 0:
            raise Unavailable("cudaEventCreate failed")
        return e

    def record(self, e) -> None:
        self.rt.cudaEventRecord(e, ctypes.c_void_p(0))

    def elapsed_ms(self, a, b) -> float:
        self.rt.cudaEventSynchronize(b)
        ms = ctypes.c_float()
        self.rt.cudaEventElapsedTime(ctypes.byref(ms), a, b)
        return float(ms.value)

    def sync(self) -> None:
        self.rt.cudaDeviceSynchronize()


def tensor_names(cfg: dict):
    """(name, shape) of every tensor the reference binds (kernels/gollmgo_model.cu:462-473,
    565-586, 708-710, 731-750, 771-773)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    d = cfg.get("head_dim") or H // nh
    yield "model.embed_tokens.weight", (V, H)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        yield p + "input_layernorm.weight", (H,)
        yield p + "self_attn.q_proj.weight", (nh * d, H)
        yield p + "self_attn.k_proj.weight", (nkv * d, H)
        yield p + "self_attn.v_proj.weight", (nkv * d, H)
        yield p + "self_attn.o_proj.weight", (H, nh * d)
        yield p + "post_attention_layernorm.weight", (H,)
        yield p + "mlp.gate_proj.weight", (I, H)
        yield p + "mlp.up_proj.weight", (I, H)
        yield p + "mlp.down_proj.weight", (H, I)
    yield "model.norm.weight", (H,)
    yield "lm_head.weight", (V, H)


def load_random_weights(ref: Reference, cfg: dict, seed: int = 0, std: float = 0.02) -> None:
    """Normal(0, std) matrices and unit norm weights in bfloat16.  Drawing 8 billion normals on
    the host takes minutes, so the matrices are windows into one pool of 2^27 draws, each
    tensor at an offset of its own: what a step costs does not depend on the values."""
    rng = np.random.default_rng(seed)
    pool = to_bf16_bits(rng.standard_normal(1 << 27, dtype=np.float32) * std)
    one = to_bf16_bits(np.ones(1, dtype=np.float32))[0]
    for i, (name, shape) in enumerate(tensor_names(cfg)):
        n = int(np.prod(shape))
        if len(shape) == 1:
            ref.load(name, np.full(n, one, dtype=np.uint16))
            continue
        off = (i * 7919 * 4099) % len(pool)
        reps = -(-(off + n) // len(pool))
        bits = pool if reps == 1 else np.tile(pool, reps)
        ref.load(name, bits[off:off + n])


def run_bench(cfg: dict, batch: int, context: int, steps: int, warmup: int, prefill_tokens: int,
              points=(1, 64), clock_sampler=None, log=None) -> dict:
    """The headline workload on the reference: ``batch`` sequences prefilled to ``context``
    tokens, then warmup + steps decode steps, every context equal and growing by one a step."""
    say = (lambda m: print(f"[reference] {m}", file=sys.stderr, flush=True)) if log is None else log
    rng = np.random.default_rng(1)
    V = cfg["vocab_size"]
    max_b = max([batch, *points])
    room = context + warmup + steps + 8
    per_seq = -(-room // 16) * 16
    max_seq_len = max(4096, -(-(room + 1) // 512) * 512)
    # kernels/gollmgo_model.cu:496-497 sizes its logits buffers with 32-bit products of
    # max_seq_len and the vocabulary
    if max_seq_len * V * 2 >= 2 ** 31:
        raise Unavailable(f"max_seq_len {max_seq_len} x vocab {V} overflows the reference's 32-bit buffer sizes")
    ref = Reference(cfg, max_seq_len, num_slots=max_b * per_seq)
    say(f"loading random weights ({cfg['num_hidden_layers']} layers)")
    load_random_weights(ref, cfg)
    ref.ready()
    big = np.empty((prefill_tokens, V), dtype=np.float32)
    logits = np.empty((max_b, V), dtype=np.float32)

    def prefill(seq: int, n: int):
        toks = rng.integers(0, V, n, dtype=np.int32)
        ref.prefill(toks, np.arange(n, dtype=np.int32), seq * per_seq + np.arange(n, dtype=np.int32), big[:n])
        return int(big[n - 1].argmax())

    # ---- prefill of prefill_tokens in one call (the last sequence's slots are used and overwritten later)
    say("prefill")
    prefill(max_b - 1, prefill_tokens)                      # warm-up: cuBLAS picks its kernels
    a, b = ref.event(), ref.event()
    reps = 2
    ref.sync()
    ref.record(a)
    for _ in range(reps):
        prefill(max_b - 1, prefill_tokens)
    ref.record(b)
    pf_ms = ref.elapsed_ms(a, b) / reps

    def decode_run(nseq: int, nsteps: int, nwarm: int, sample_clocks: bool):
        next_tok = np.array([prefill(s, context) for s in range(nseq)], dtype=np.int32)
        ctx = context
        table = np.zeros((nseq, context + nwarm + nsteps + 1), dtype=np.int32)
        for s in range(nseq):
            table[s] = s * per_seq + np.arange(table.shape[1])

        def one():
            nonlocal ctx, next_tok
            pos = np.full(nseq, ctx, dtype=np.int32)
            ref.decode(next_tok, pos, table[:, ctx], pos + 1, table[:, :ctx + 1], logits[:nseq])
            next_tok = logits[:nseq].argmax(axis=1).astype(np.int32)       # greedy, on the host
            ctx += 1
        for _ in range(nwarm):
            one()
        clocks = clock_sampler() if (sample_clocks and clock_sampler) else None
        if clocks:
            clocks.start()
        ref.sync()
        t0 = time.perf_counter()
        ref.record(a)
        for _ in range(nsteps):
            one()
        ref.record(b)
        ms = ref.elapsed_ms(a, b)
        wall = time.perf_counter() - t0
        c = clocks.stop() if clocks else None
        if not np.isfinite(logits[:nseq]).all():
            raise Unavailable("the reference produced non-finite logits")
        return ms / nsteps, wall / nsteps, c

    say(f"decode, batch {batch}")
    ms_step, wall_step, clocks = decode_run(batch, steps, warmup, True)
    pts = {}
    for p in points:
        if p == batch:
            continue
        say(f"decode, batch {p}")
        pts[f"decode_b{p}"] = round(p / (decode_run(p, min(steps, 32), 3, False)[0] / 1e3), 1)
    ref.close()
    return {"ms_per_step": ms_step, "wall_per_step": wall_step, "clocks": clocks, "prefill_ms": pf_ms,
            "points": pts, "max_seq_len": max_seq_len,
            "h2d_bytes_per_step": int(4 * (4 * batch + batch * (context + warmup + steps // 2))),
            "d2h_bytes_per_step": int(4 * batch * V)}


def run_anchor(in_npz: str, out_npz: str) -> None:
    """A tiny model through the reference, for pinning a plain implementation on its output.
    ``in_npz`` holds ``config`` (JSON text), every weight as bfloat16 bit patterns under its
    tensor name, ``tokens`` and ``n_prefill``.  Written to ``out_npz``: ``whole`` = logits of
    all tokens from one gollmgo_model_forward call; ``paged`` = logits of the last prompt token
    from gollmgo_model_forward_prefill over the first n_prefill tokens followed by one
    gollmgo_model_forward_paged call per remaining token (one sequence, slots scattered)."""
    data = np.load(in_npz)
    cfg = json.loads(str(data["config"]))
    tokens = data["tokens"].astype(np.int32)
    n_pre = int(data["n_prefill"])
    T, V = len(tokens), cfg["vocab_size"]
    ref = Reference(cfg, max_seq_len=512, num_slots=256)
    for name, _ in tensor_names(cfg):
        ref.load(name, data[name])
    ref.ready()
    whole = np.empty((T, V), dtype=np.float32)
    ref.forward(tokens, np.arange(T, dtype=np.int32), whole)
    slots = np.random.default_rng(3).permutation(256)[:T].astype(np.int32)      # any slots will do
    pre = np.empty((n_pre, V), dtype=np.float32)
    ref.prefill(tokens[:n_pre], np.arange(n_pre, dtype=np.int32), slots[:n_pre], pre)
    rows = [pre[n_pre - 1].copy()]
    one = np.empty((1, V), dtype=np.float32)
    for t in range(n_pre, T):
        ref.decode(tokens[t:t + 1], [t], slots[t:t + 1], [t + 1], slots[None, :t + 1], one)
        rows.append(one[0].copy())
    ref.close()
    np.savez(out_npz, whole=whole, paged=np.stack(rows), prefill=pre)


if __name__ == "__main__":
    if len(sys.argv) == 4 and sys.argv[1] == "anchor":
        run_anchor(sys.argv[2], sys.argv[3])
    else:
        print(build(verbose=True))
