"""Measured comparators for the decode step.  Never a dispatch target: the engine does not import this module.

The reference's README compares its kernel with general-purpose stacks on the same step (README.md:12-18:
FlashInfer, torch.compile, cuBLAS through PyTorch under a CUDA graph).  The one of those that needs nothing but
PyTorch is kept here as `TorchGraphDecoder`: the decode step written with stock torch ops on the bf16 weights
(matrix-vector products go to cuBLAS), captured once in a CUDA graph and replayed, so that what is timed is kernel
time and not Python.  `compare` times it next to the engine on the same inputs.
"""
from __future__ import annotations

import statistics

import torch

from .kernel import HEAD_DIM, KV_HEADS, Q_HEADS, Megakernel, rope_table

EPS = 1e-6


class TorchGraphDecoder:
    """Batch-1 decode at a fixed position with torch ops, replayed from a CUDA graph.  bf16 weights and bf16 matrix
    products with fp32 norms, softmax and residual stream (the usual mixed-precision recipe); the new K/V row enters
    attention unrounded, like the engine's.  products="fp32" widens the weights and keeps every product in fp32: slower,
    and an implementation of the step that shares no code with the engine, which `run.py check` gates the kernels on."""

    def __init__(self, inputs: dict, products: str = "bf16"):
        self.act = torch.bfloat16 if products == "bf16" else torch.float32
        self.w = inputs if products == "bf16" else {k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in inputs.items()}
        dev = inputs["embed"].device
        self.device = dev
        self.layers = inputs["wq"].shape[0]
        self.ctx = inputs["kcache"].shape[1]
        rope = rope_table(dev, self.ctx)
        self.cos, self.sin = torch.cat([rope[:64], rope[:64]]), torch.cat([rope[64:], rope[64:]])
        self.kf = inputs["kcache"].float()      # [L, ctx, 8, 128]
        self.vf = inputs["vcache"].float()
        self.token = inputs["token"].clone()
        self.k_write = torch.empty((self.layers, KV_HEADS, HEAD_DIM), dtype=torch.float32, device=dev)
        self.v_write = torch.empty_like(self.k_write)
        self.logits = torch.empty(inputs["embed"].shape[0], dtype=torch.float32, device=dev)
        self.next_token = torch.empty((), dtype=torch.int64, device=dev)
        self.graph = None

    @staticmethod
    def _rms(x, gain):
        return (x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + EPS)) * gain.float()

    def _rot(self, x):
        return x * self.cos + torch.cat([-x[..., 64:], x[..., :64]], dim=-1) * self.sin

    def _step(self):
        w = self.w
        x = torch.index_select(w["embed"], 0, self.token.reshape(1))[0].float()   # (indexing by a device scalar would synchronise)
        for l in range(self.layers):
            xn = self._rms(x, w["ln1"][l]).to(self.act)
            q = (w["wq"][l] @ xn).float().view(Q_HEADS, HEAD_DIM)
            k = (w["wk"][l] @ xn).float().view(KV_HEADS, HEAD_DIM)
            v = (w["wv"][l] @ xn).float().view(KV_HEADS, HEAD_DIM)
            q = self._rot(self._rms(q, w["qn"][l]))
            k = self._rot(self._rms(k, w["kn"][l]))
            self.k_write[l].copy_(k)
            self.v_write[l].copy_(v)
            ka = torch.cat([self.kf[l], k[None]], dim=0).repeat_interleave(Q_HEADS // KV_HEADS, dim=1)   # [ctx + 1, 16, 128]
            va = torch.cat([self.vf[l], v[None]], dim=0).repeat_interleave(Q_HEADS // KV_HEADS, dim=1)
            s = torch.einsum("hd,shd->hs", q, ka) * HEAD_DIM ** -0.5
            o = torch.einsum("hs,shd->hd", torch.softmax(s, dim=-1), va).reshape(-1)
            x = x + (w["wo"][l] @ o.to(self.act)).float()
            xn = self._rms(x, w["ln2"][l]).to(self.act)
            h = torch.nn.functional.silu((w["wg"][l] @ xn).float()) * (w["wu"][l] @ xn).float()
            x = x + (w["wd"][l] @ h.to(self.act)).float()
        self.logits.copy_((w["embed"] @ self._rms(x, w["fnorm"]).to(self.act)).float())
        self.next_token.copy_(self.logits.argmax())

    @torch.no_grad()
    def capture(self):
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(3):
                self._step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step()
        return self

    def launch(self):
        self.graph.replay()


def _time(launch, steps: int, reps: int, device) -> dict:
    per = []
    for _ in range(reps):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            launch()
        t1.record()
        torch.cuda.synchronize(device)
        per.append(t0.elapsed_time(t1) * 1e3 / steps)
    return {"us_per_step_median": statistics.median(per), "us_per_step_min": min(per)}


def compare(inputs: dict, steps: int = 50, reps: int = 5) -> list[dict]:
    """Rows {name, us_per_step_median, us_per_step_min, note}: the engine's persistent kernel, its layered path under graph
    replay, and cuBLAS through PyTorch under a CUDA graph, all on `inputs` (batch 1, position = the cache length)."""
    dev = inputs["embed"].device
    rows = []
    for path in ("persist", "layered"):
        mk = Megakernel(dev, layers=inputs["wq"].shape[0], vocab=inputs["embed"].shape[0], path=path)
        out = mk.bind(inputs)
        for _ in range(20):
            mk.launch()
        torch.cuda.synchronize(dev)
        r = _time(mk.launch, steps, reps, dev)
        mk.status()
        if path == "persist":
            ours = {k: v.clone() for k, v in out.items()}
        rows.append({"name": f"this engine, {path} path", **r, "note": "fp32 activations, bf16 weights"})
    base = TorchGraphDecoder(inputs).capture()
    base.launch()
    torch.cuda.synchronize(dev)
    r = _time(base.launch, steps, reps, dev)
    err = float((base.logits.double() - ours["logits"].double()).norm() / ours["logits"].double().norm())
    rows.append({"name": "cuBLAS through PyTorch, CUDA graph", **r,
                 "note": f"bf16 products; logits rel-L2 to the engine {err:.1e}, token {'equal' if int(base.next_token) == int(ours['next_token']) else 'differs'}"})
    return rows
