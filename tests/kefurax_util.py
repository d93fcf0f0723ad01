"""Small random Kefurax checkpoints for the tests: configuration builders and seeded weights (values representable in
bfloat16, so that both storage types and the float64 oracle read the same numbers).  The safetensors writer is the one of
tests/pikavik_util.py."""
from __future__ import annotations

import math

import torch

from tests.pikavik_util import rel_err, write_checkpoint  # noqa: F401  (re-exported)
from tests import kefurax_plain as P


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def rglru(width=24, blocks=2, conv=4, mlp=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def mamba1(inner=20, state=6, dt_rank=3, conv=3, mlp=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def attention(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.4, dims=4, base=1000.0, scaling="default"):
    rot = None
    if dims:
        rot = {"base": base, "dims": dims}
        if scaling == "default":
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
        elif scaling:
            rot["scaling"] = scaling
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        a["rot"] = rot
    return a


def delta(heads=4, kv_heads=2, dim=6, vdim=5, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(left=None, right=None, left_scale=0.7, right_scale=1.2, mlp=None):
    return {"type": "parallel", "mixer": {"left": left or attention(), "right": right or delta(), "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def config(layers, width=40, vocab=50, eps=1e-5, mult=0.6, embed_scale=2.5):
    return {"architecture": "Kefurax", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
            "residual_mult": mult, "vocab": vocab, "width": width}


def random_tensors(cfg: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def lin(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g)

    def uni(shape, lo, hi):
        return lo + (hi - lo) * torch.rand(shape, generator=g)

    t = {"embed": torch.randn(cfg["vocab"], W, generator=g), "head": lin(cfg["vocab"], W), "final.norm": vec(W, 1.0)}
    for i, lc in enumerate(cfg["layers"]):
        p, mx, m = f"l{i}.", f"l{i}.mix.", lc["mixer"]
        t[p + "norm1"] = vec(W, 1.0)
        if lc["type"] == "rglru":
            R, nb, taps = m["width"], m["blocks"], m["conv"]
            bs = R // nb
            t[mx + "y"], t[mx + "y.b"], t[mx + "x"], t[mx + "x.b"] = lin(R, W), vec(R, 0.0, 0.3), lin(R, W), vec(R, 0.0, 0.3)
            t[mx + "conv"], t[mx + "conv.b"] = torch.randn(R, taps, generator=g) * 0.5, vec(R, 0.0, 0.2)
            t[mx + "ra"], t[mx + "ri"] = torch.randn(nb, bs, bs, generator=g) / bs ** 0.5, torch.randn(nb, bs, bs, generator=g) / bs ** 0.5
            t[mx + "ra.b"], t[mx + "ri.b"] = torch.randn(nb, bs, generator=g) * 0.5, torch.randn(nb, bs, generator=g) * 0.5
            t[mx + "lam"], t[mx + "o"] = uni(R, -4.0, 0.5), lin(W, R)
        elif lc["type"] == "mamba1":
            I, N, Rk, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
            t[mx + "in"], t[mx + "conv"], t[mx + "conv.b"] = lin(2 * I, W), torch.randn(I, taps, generator=g) * 0.5, vec(I, 0.0, 0.2)
            t[mx + "x"], t[mx + "dt"], t[mx + "dt.b"] = lin(Rk + 2 * N, I, 2.0), lin(I, Rk), uni(I, -3.0, -0.5)
            t[mx + "A_log"], t[mx + "D"], t[mx + "o"] = torch.log(uni((I, N), 0.3, 4.0)), vec(I, 1.0, 0.2), lin(W, I)
        else:
            a, d = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = mx + "left."
            t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"], t[q + "o"] = lin(H * D, W), lin(G * D, W), lin(G * V, W), lin(H * V, W), lin(W, H * V)
            H, G, D, V, taps = d["heads"], d["kv_heads"], d["dim"], d["vdim"], d["conv"]
            q = mx + "right."
            t[q + "q"], t[q + "k"], t[q + "v"] = lin(G * D, W, 2.0), lin(G * D, W, 2.0), lin(H * V, W, 2.0)
            for s, c in (("q", G * D), ("k", G * D), ("v", H * V)):
                t[f"{q}{s}.conv"] = torch.randn(c, taps, generator=g) * 0.6
            t[q + "b"], t[q + "a"], t[q + "g"], t[q + "o"] = lin(H, W, 2.0), lin(H, W, 2.0), lin(H * V, W), lin(W, H * V)
            t[q + "A_log"], t[q + "dt_bias"], t[q + "norm"] = uni(H, -2.0, 0.5), uni(H, -2.0, 1.0), vec(V, 1.0)
        if lc.get("mlp"):
            ff = lc["mlp"]["ff"]
            t[p + "norm2"] = vec(W, 1.0)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}


class PlainModel:
    """The oracle over raw tensors: whole prompts, portions (through a carried state) and greedy continuation."""

    def __init__(self, cfg, tensors):
        self.cfg, self.W = cfg, {k: v.to(torch.float64) for k, v in tensors.items()}

    def run(self, tokens, layers_out=None, state=None, p0=0):
        logits, taps = P.forward(self.cfg, self.W, list(tokens), {} if state is None else state, p0)
        if layers_out is not None:
            layers_out.extend(taps)
        return logits

    def greedy(self, prompt, n):
        state, out = {}, []
        logits = self.run(prompt, state=state)
        pos = len(prompt)
        for _ in range(n):
            tok = int(torch.argmax(logits[-1]))
            out.append(tok)
            logits = self.run([tok], state=state, p0=pos)
            pos += 1
        return out
