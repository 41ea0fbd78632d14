"""Host side of the decode engine: load libq3mk.so and launch decode steps.

Mirrors the operator API of the reference's launcher (qwen3mk/kernel.py:109-233): `Megakernel` with
`step`, `bind`, `launch`, `chain_token` and `check_inputs`, the tuples `INPUT_ORDER`, `INPUT_SPECS`,
`OUTPUT_SPECS`, and `rope_table`.  The reference JIT-compiles one fixed-shape kernel with NVRTC; here
the kernels are prebuilt for sm_100a and reached through the C ABI in include/q3mk.h, and the fixed
case (batch 1, position 128) is one point of a general one:

  * the position is the cache length: `kcache.shape[1]` (any length, not only 128);
  * `SeqTable` + `bind_sequences` decode a batch of sequences with their own lengths and caches;
  * with `append=True` the engine writes each new K/V row into the sequence's cache and advances its
    length on the device, so chained launches walk forward without host work.

As in the reference the engine never synchronises, never validates in `step`, borrows every tensor
it is given and never writes to an input (the caches are written only when `append=True`).
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi

INPUT_ORDER = ("token", "ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2",
               "wg", "wu", "wd", "fnorm", "embed", "kcache", "vcache")
WEIGHT_ORDER = _cabi.WEIGHT_FIELDS

LAYERS, HIDDEN, Q_HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB, CONTEXT = 28, 1024, 16, 8, 128, 3072, 151936, 128
ROPE_THETA = 1e6
EXPECTED_PARAMS = {"batch": "1..max_batch", "context": "any (cache length)", "layers": LAYERS, "hidden": HIDDEN,
                   "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": HEAD_DIM, "intermediate": INTER, "vocab": VOCAB}


def input_specs(layers: int = LAYERS, vocab: int = VOCAB, context: int = CONTEXT) -> dict:
    """Shape and dtype of every input for a model of `layers` layers and `vocab` words at cache length `context`."""
    bf = torch.bfloat16
    return {
        "token": ((), torch.int64),
        "ln1": ((layers, HIDDEN), bf),
        "wq": ((layers, Q_HEADS * HEAD_DIM, HIDDEN), bf),
        "wk": ((layers, KV_HEADS * HEAD_DIM, HIDDEN), bf),
        "wv": ((layers, KV_HEADS * HEAD_DIM, HIDDEN), bf),
        "qn": ((layers, HEAD_DIM), bf),
        "kn": ((layers, HEAD_DIM), bf),
        "wo": ((layers, HIDDEN, Q_HEADS * HEAD_DIM), bf),
        "ln2": ((layers, HIDDEN), bf),
        "wg": ((layers, INTER, HIDDEN), bf),
        "wu": ((layers, INTER, HIDDEN), bf),
        "wd": ((layers, HIDDEN, INTER), bf),
        "fnorm": ((HIDDEN,), bf),
        "embed": ((vocab, HIDDEN), bf),
        "kcache": ((layers, context, KV_HEADS, HEAD_DIM), bf),
        "vcache": ((layers, context, KV_HEADS, HEAD_DIM), bf),
    }


def output_specs(layers: int = LAYERS, vocab: int = VOCAB) -> dict:
    return {
        "logits": ((vocab,), torch.float32),
        "next_token": ((), torch.int64),
        "k_write": ((layers, KV_HEADS, HEAD_DIM), torch.bfloat16),
        "v_write": ((layers, KV_HEADS, HEAD_DIM), torch.bfloat16),
    }


# the reference's fixed case, under the reference's names
INPUT_SPECS = input_specs()
OUTPUT_SPECS = output_specs()


def rope_rows(n_positions: int, device) -> torch.Tensor:
    """RoPE table fp32 [n_positions, 128]: row p is cos(p*f) for the 64 frequencies, then sin(p*f); fp64 math."""
    freq = ROPE_THETA ** (-torch.arange(0, HEAD_DIM, 2, dtype=torch.float64) / HEAD_DIM)
    ang = torch.arange(n_positions, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).float().contiguous().to(device)


def rope_table(device, position: int = CONTEXT) -> torch.Tensor:
    """cos then sin at one position, fp32 [128] (the reference's table; qwen3mk/kernel.py:102-106)."""
    freq = ROPE_THETA ** (-torch.arange(0, HEAD_DIM, 2, dtype=torch.float64) / HEAD_DIM)
    ang = float(position) * freq
    return torch.cat([ang.cos(), ang.sin()]).float().to(device)


class SeqTable:
    """Device-resident descriptors of a batch of sequences: cache addresses, layer strides, lengths.

    kcaches / vcaches: one bf16 tensor [layers, capacity_b, 8, 128] per sequence (contiguous).
    lens: cached positions per sequence (default: the full capacity).  The engine reads these arrays
    on the device; with `append=True` it also advances `len` there."""

    def __init__(self, kcaches, vcaches, lens=None, device=None):
        if len(kcaches) != len(vcaches) or not kcaches:
            raise ValueError("SeqTable: need one K and one V cache per sequence")
        device = kcaches[0].device if device is None else torch.device(device)
        caps = []
        for k, v in zip(kcaches, vcaches):
            for t in (k, v):
                if (t.dim() != 4 or tuple(t.shape[2:]) != (KV_HEADS, HEAD_DIM) or t.dtype != torch.bfloat16
                        or not t.is_contiguous() or t.device != device):
                    raise ValueError(f"SeqTable: expected contiguous bf16 [layers, capacity, 8, 128] on {device}, "
                                     f"got {t.dtype} {tuple(t.shape)} on {t.device}")
            if k.shape != v.shape:
                raise ValueError("SeqTable: K and V cache shapes differ")
            caps.append(int(k.shape[1]))
        lens = caps if lens is None else [int(x) for x in lens]
        if len(lens) != len(caps) or any(n < 0 or n > c for n, c in zip(lens, caps)):
            raise ValueError("SeqTable: every length must lie in [0, capacity]")
        self.kcaches, self.vcaches = list(kcaches), list(vcaches)   # keep the memory alive
        self.capacity = caps
        self.host_len = list(lens)
        self.batch = len(caps)
        i64 = torch.int64
        self.seq_k = torch.tensor([t.data_ptr() for t in kcaches], dtype=i64).to(device)
        self.seq_v = torch.tensor([t.data_ptr() for t in vcaches], dtype=i64).to(device)
        self.stride = torch.tensor([c * KV_HEADS * HEAD_DIM for c in caps], dtype=i64).to(device)
        self.len = torch.tensor(lens, dtype=torch.int32).to(device)

    @property
    def max_len(self) -> int:
        return max(self.host_len)


class Megakernel:
    """The decode engine on one GPU.

    `step(inputs)` runs one batch-1 decode step at position `kcache.shape[1]` and returns a dict with
    `logits`, `next_token`, `k_write`, `v_write`.  `bind(inputs)` + `launch(stream)` is the low-level
    path: fixed inputs, outputs overwritten by every launch, no synchronisation.
    `bind_sequences` is the batched / growing-cache form of `bind`.

    path: "auto" (persistent kernel when it serves the batch, else layered), "layered" (one launch per phase), "fused" (layered, with
    one persistent kernel for everything between two attentions for batches of 4..64; opt-in) or "persist".
    """

    def __init__(self, device=None, *, max_batch: int = 1, layers: int = LAYERS, vocab: int = VOCAB,
                 max_positions: int = 8192, path: str = "auto", grid_limit: int = 0, max_tokens: int = 0,
                 wait_limit_us: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("Megakernel needs a CUDA device (sm_100a); there is no CPU path")
        self.lib = _cabi.load()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError(f"Megakernel needs a CUDA device, got {self.device}")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        torch.zeros(1, device=self.device)  # make torch's primary context current
        major, minor = torch.cuda.get_device_capability(self.device)
        self.arch = f"sm_{major}{minor}"
        self.layers, self.vocab, self.max_batch = int(layers), int(vocab), int(max_batch)
        self._path_flag = {"auto": _cabi.F_PATH_AUTO, "layered": _cabi.F_PATH_LAYERED, "persist": _cabi.F_PATH_PERSIST,
                           "fused": _cabi.F_PATH_FUSED}[path]
        cfg = _cabi.Config(self.layers, self.vocab, self.max_batch, int(max_tokens), int(grid_limit), int(wait_limit_us))
        h = ctypes.c_void_p()
        rc = self.lib.q3_create(self.device.index or 0, ctypes.byref(cfg), ctypes.byref(h))
        _cabi.check(self.lib, None, rc, "q3_create")
        self.handle = h
        self.rope = rope_rows(int(max_positions), self.device)
        _cabi.check(self.lib, h, self.lib.q3_set_rope(h, self.rope.data_ptr(), self.rope.shape[0]), "q3_set_rope")
        g, t, s = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        self.lib.q3_grid_info(h, ctypes.byref(g), ctypes.byref(t), ctypes.byref(s))
        self.grid, self.threads, self.dyn_smem = g.value, t.value, s.value
        self._out_specs = output_specs(self.layers, self.vocab)
        self._weights_key = None
        self._weights_ref = None
        self.tp = None           # the rank's tensor-parallel share (qwen3mk.tp.attach), or None
        self._seq_cache = {}     # step(): descriptors per (kcache ptr, vcache ptr, context)
        self._next = None        # step(): outputs of the next call, allocated while the kernel runs
        self._bound = None
        self._args = _cabi.DecodeArgs()
        self._out = None
        self._tok = None
        self._n_launch = 0
        self._chained = False
        self._append = False
        self._max_launches = None
        self._base_len = 0

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                self.lib.q3_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # ------------------------------------------------------------------ helpers

    def _alloc(self, batch: int | None = None):
        dev = self.device
        lead = () if batch is None else (batch,)
        return tuple(torch.empty(lead + shape, dtype=dt, device=dev) for shape, dt in self._out_specs.values())

    def _set_weights(self, inputs: dict) -> None:
        """Hand the 13 weight pointers to the engine when they, or the tensors' contents, have changed.

        The persistent kernel streams an engine-owned re-layout of the layer matrices, so a change that keeps the
        addresses must still reach the engine: the key holds every tensor's version counter (PyTorch bumps it on
        every in-place write), and the engine keeps references to the tensors it packed, so that their memory cannot
        be freed and handed out again, with other contents, at the same addresses."""
        tensors = tuple(inputs[n] for n in WEIGHT_ORDER)
        key = tuple((t.data_ptr(), t._version) for t in tensors)
        if key == self._weights_key:
            return
        ptrs = tuple(k[0] for k in key)
        if self._weights_key is not None and ptrs == tuple(k[0] for k in self._weights_key):
            self.lib.q3_invalidate_weights(self.handle)    # same addresses, rewritten in place
        w = _cabi.Weights(*ptrs)
        _cabi.check(self.lib, self.handle, self.lib.q3_set_weights(self.handle, ctypes.byref(w)), "q3_set_weights")
        self._weights_key = key
        self._weights_ref = tensors

    def refresh_weights(self) -> None:
        """Forget the engine's packed copy of the layer matrices.  Only needed after a write that PyTorch's version
        counters do not see (a raw-pointer write from another library): in-place tensor operations are noticed."""
        self.lib.q3_invalidate_weights(self.handle)
        self._weights_key = None

    def check_inputs(self, inputs: dict) -> None:
        """Raise ValueError unless every input is a contiguous CUDA tensor of the expected shape and dtype."""
        ctx = inputs["kcache"].shape[1] if "kcache" in inputs and inputs["kcache"].dim() == 4 else CONTEXT
        specs = input_specs(self.layers, self.vocab, ctx)
        for name in INPUT_ORDER:
            t = inputs[name]
            shape, dt = specs[name]
            if tuple(t.shape) != shape or t.dtype != dt or not t.is_contiguous() or not t.is_cuda:
                raise ValueError(f"input {name}: expected a contiguous CUDA tensor {dt} {shape}, got {t.dtype} {tuple(t.shape)}")

    def status(self, stream=None) -> list[int]:
        """Synchronise and read the device status words; raises RuntimeError if a device-side wait gave up."""
        words = (ctypes.c_uint32 * 8)()
        st = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        rc = self.lib.q3_status(self.handle, st, words, 8)
        _cabi.check(self.lib, self.handle, rc, "q3_status")
        return list(words)

    @property
    def launch_count(self) -> int:
        """Kernels this engine has launched since creation."""
        return int(self.lib.q3_launch_count(self.handle))

    def scratch(self, name: str, view: bool = False) -> torch.Tensor:
        """An engine scratch buffer ("x", "qkv", "attn", "hid", "status", "persist_acc") as a float32 tensor, for tools
        and tests: a copy, or with view=True the engine's own memory (valid while the engine lives)."""
        p, n = ctypes.c_void_p(), ctypes.c_int64()
        rc = self.lib.q3_scratch(self.handle, name.encode(), ctypes.byref(p), ctypes.byref(n))
        _cabi.check(self.lib, self.handle, rc, "q3_scratch")
        class _Raw:  # expose the engine's buffer to torch through the CUDA array interface
            __cuda_array_interface__ = {"shape": (n.value // 4,), "typestr": "<f4", "data": (p.value, False), "version": 3}
        torch.cuda.synchronize(self.device)
        t = torch.as_tensor(_Raw(), device=self.device)
        return t if view else t.clone()

    def enable_trace(self, on: bool = True):
        """Phase time stamps of the persistent kernel: returns the int64 device tensor [grid, 4 + 12 * layers]
        that every later persistent launch overwrites with %globaltimer values (ns), or None when switched off."""
        if not on or self.grid == 0:
            self._trace = None
            self.lib.q3_set_trace(self.handle, None, 0)
            return None
        self._trace = torch.zeros((self.grid, 4 + 12 * self.layers), dtype=torch.int64, device=self.device)
        rc = self.lib.q3_set_trace(self.handle, self._trace.data_ptr(), self._trace.numel())
        _cabi.check(self.lib, self.handle, rc, "q3_set_trace")
        return self._trace

    def _decode(self, args, stream) -> None:
        rc = self.lib.q3_decode(self.handle, ctypes.byref(args), stream)
        _cabi.check(self.lib, self.handle, rc, "q3_decode")

    # ------------------------------------------------------------------ step

    def step(self, inputs: dict) -> dict:
        """One batch-1 decode step at position `kcache.shape[1]`.  Enqueues on the current stream and
        returns fresh tensors that no later call writes (the next call's outputs are allocated right
        after the launch, while the kernel runs; qwen3mk/kernel.py:180-191)."""
        logits, next_token, k_write, v_write = self._next if self._next is not None else self._alloc()
        self._set_weights(inputs)
        kc, vc = inputs["kcache"], inputs["vcache"]
        key = (kc.data_ptr(), vc.data_ptr(), kc.shape[1])
        seqs = self._seq_cache.get(key)
        if seqs is None:
            if len(self._seq_cache) > 64:
                self._seq_cache.clear()
            seqs = self._seq_cache[key] = SeqTable([kc], [vc], device=self.device)
        a = _cabi.DecodeArgs(1, seqs.max_len, self._path_flag, 0, inputs["token"].data_ptr(), seqs.seq_k.data_ptr(),
                             seqs.seq_v.data_ptr(), seqs.stride.data_ptr(), seqs.len.data_ptr(), logits.data_ptr(),
                             next_token.data_ptr(), k_write.data_ptr(), v_write.data_ptr())
        self._decode(a, torch.cuda.current_stream(self.device).cuda_stream)
        self._next = self._alloc()
        return {"logits": logits, "next_token": next_token, "k_write": k_write, "v_write": v_write}

    # ------------------------------------------------------------------ bound path

    def bind(self, inputs: dict, chained: bool = False, grow: int = 0) -> dict:
        """Fix the inputs for `launch`; returns the output tensors every launch overwrites.

        chained=True: the token comes from a device buffer that the previous launch wrote (two buffers
        swap on every launch; the last token is `chain_token`).  grow=N (N > 0): the engine keeps its own
        copy of the caches with room for N more positions and appends each step's K/V rows, so launch i
        decodes position context+i; the caller's tensors stay untouched.  grow=0 is the reference's
        behaviour: every launch decodes the same position (qwen3mk/kernel.py:195-213)."""
        self.check_inputs(inputs)
        kc, vc = inputs["kcache"], inputs["vcache"]
        ctx = kc.shape[1]
        if grow > 0:
            room = (self.layers, ctx + grow, KV_HEADS, HEAD_DIM)
            kbuf = torch.zeros(room, dtype=torch.bfloat16, device=self.device)
            vbuf = torch.zeros(room, dtype=torch.bfloat16, device=self.device)
            kbuf[:, :ctx] = kc
            vbuf[:, :ctx] = vc
            seqs = SeqTable([kbuf], [vbuf], [ctx], device=self.device)
        else:
            seqs = SeqTable([kc], [vc], device=self.device)
        out = self.bind_sequences(inputs, inputs["token"].reshape(1), seqs, append=grow > 0, chained=chained)
        self._bound = ({k: inputs[k] for k in INPUT_ORDER}, seqs)
        self._out = tuple(t[0] for t in self._out)
        return dict(zip(self._out_specs, self._out))

    def bind_sequences(self, weights: dict, tokens: torch.Tensor, seqs: SeqTable, *, append: bool = False,
                       chained: bool = False, want_logits: bool = True, graph: bool = True) -> dict:
        """Batched form of `bind`: `tokens` int64 [B] on the device, `seqs` a SeqTable of B sequences.
        Returns outputs with a leading batch axis.  With append=True each launch writes the new K/V rows
        into the caches and advances the device-side lengths (capacity is the caller's responsibility:
        at most capacity_b - len_b launches).  graph=False keeps the layered path on plain launches
        (one per kernel), which is what a profiler wants to see."""
        B = seqs.batch
        if tokens.dtype != torch.int64 or tokens.numel() != B or not tokens.is_cuda or not tokens.is_contiguous():
            raise ValueError(f"tokens: expected a contiguous CUDA int64 tensor of {B} elements")
        if B > self.max_batch:
            raise ValueError(f"batch {B} exceeds max_batch {self.max_batch} of this engine")
        self._set_weights(weights)
        self._bound = (weights, seqs)
        self._out = self._alloc(B)
        logits, next_token, k_write, v_write = self._out
        # bound launches repeat the same argument block: let the layered path replay a CUDA graph
        flags = self._path_flag | (_cabi.F_APPEND_KV if append else 0) | (_cabi.F_GRAPH if graph else 0)
        self._args = _cabi.DecodeArgs(B, seqs.max_len, flags, 0, tokens.data_ptr(), seqs.seq_k.data_ptr(),
                                      seqs.seq_v.data_ptr(), seqs.stride.data_ptr(), seqs.len.data_ptr(),
                                      logits.data_ptr() if want_logits else None, next_token.data_ptr(),
                                      k_write.data_ptr(), v_write.data_ptr())
        self._chained, self._append = chained, append
        self._n_launch = 0
        self._base_len = seqs.max_len
        self._max_launches = min(c - n for c, n in zip(seqs.capacity, seqs.host_len)) if append else None
        self._tok = (tokens.clone(), torch.zeros_like(tokens)) if chained else (tokens, None)
        return dict(zip(self._out_specs, self._out))

    @property
    def chain_token(self) -> torch.Tensor:
        """The token(s) the next chained launch reads (the argmax of the last one)."""
        t = self._tok[self._n_launch & 1]
        return t[0] if t.numel() == 1 else t

    def launch(self, stream=None) -> None:
        """Enqueue one decode step on the bound inputs.  No host sync.  `stream` is a CUDA stream handle (int)."""
        if self._bound is None:
            raise RuntimeError("call bind(inputs) before launch()")
        a = self._args
        if self._append:
            if self._n_launch >= self._max_launches:
                raise RuntimeError("launch(): the bound caches are full")
            a.max_len = self._base_len + self._n_launch
        if self._chained:
            a.token = self._tok[self._n_launch & 1].data_ptr()
            a.next_token = self._tok[(self._n_launch + 1) & 1].data_ptr()
        self._decode(a, torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream)
        self._n_launch += 1
