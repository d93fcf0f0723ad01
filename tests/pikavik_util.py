"""Small random Pikavik checkpoints for the tests: configuration builders, seeded weights (values representable in
bfloat16, so that both storage types and the float64 oracle read the same numbers) and a minimal safetensors writer."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch


def moe(experts=6, top=3, groups=3, keep=2, ff=20, limit=1.5, scale=2.0, shared_ff=12, shared_limit=0.8):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "scale": scale, "top": top},
         "shared": {"ff": shared_ff, "limit": shared_limit} if shared_ff else None}
    return m


def wkv(heads=2, dim=12, mlp=None, rank=6):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp, "_rank": rank}


def mlstm(heads=2, dim=10, vdim=6, cap=15.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def latent(heads=3, dim=10, rot_dim=8, vdim=14, kv_rank=20, q_rank=18, scale=0.3, base=10000.0, mlp=None, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": dims or rot_dim}}, "mlp": mlp}


def config(layers, width=40, vocab=50, eps=1e-6):
    return {"architecture": "Pikavik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def random_tensors(cfg: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def lin(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g)

    def uni(n, lo, hi):
        return lo + (hi - lo) * torch.rand(n, generator=g)

    t = {"embed": torch.randn(cfg["vocab"], W, generator=g), "head": lin(cfg["vocab"], W), "final.norm": vec(W)}
    for i, lc in enumerate(cfg["layers"]):
        p, mx, m = f"l{i}.", f"l{i}.mix.", lc["mixer"]
        t[p + "norm1"], t[p + "ls1"] = vec(W), uni(W, 0.5, 1.5)
        H, D = m["heads"], m["dim"]
        if lc["type"] == "wkv":
            rank = lc.get("_rank", 6)
            for s in "rkvgw":
                t[mx + "mu." + s] = uni(W, 0.0, 1.0)
            for s in "rkvg":
                t[mx + s] = lin(H * D, W)
            t[mx + "w1"], t[mx + "w2"], t[mx + "w0"] = lin(rank, W), lin(H * D, rank), uni(H * D, -2.5, 0.5)
            t[mx + "u"], t[mx + "norm"], t[mx + "o"] = 0.5 * torch.randn(H, D, generator=g), vec(H * D, 1.0), lin(W, H * D)
        elif lc["type"] == "mlstm":
            V = m["vdim"]
            t[mx + "q"], t[mx + "k"], t[mx + "v"], t[mx + "g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[mx + "i"], t[mx + "f"] = lin(H, W, 2.0), lin(H, W, 2.0)
            t[mx + "i.b"], t[mx + "f.b"] = vec(H, 0.0, 1.0), uni(H, 1.0, 4.0)
            t[mx + "norm"], t[mx + "o"] = vec(H * V, 1.0), lin(W, H * V)
        else:
            R, V, KR, QR = m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[mx + "dq"], t[mx + "dq.norm"], t[mx + "uq"] = lin(QR, W), vec(QR, 1.0), lin(H * (D + R), QR)
            t[mx + "dkv"], t[mx + "dkv.norm"] = lin(KR + R, W), vec(KR, 1.0)
            t[mx + "uk"], t[mx + "uv"] = lin(H * D, KR), lin(H * V, KR)
            t[mx + "sink"], t[mx + "o"] = vec(H, 0.0, 1.0), lin(W, H * V)
        mlp = lc.get("mlp")
        if mlp:
            q, ff = p + "mlp.", mlp["expert"]["ff"]
            t[p + "ls2"] = uni(W, 0.5, 1.5)
            t[q + "router"] = lin(mlp["router"]["experts"], W, 3.0)
            for e in range(mlp["router"]["experts"]):
                t[f"{q}e{e}.gate"], t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
            if mlp.get("shared"):
                sff = mlp["shared"]["ff"]
                t[q + "shared.gate"], t[q + "shared.up"], t[q + "shared.down"] = lin(sff, W, 2.0), lin(sff, W, 2.0), lin(W, sff)
                t[q + "shared.sg"] = lin(1, W)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}


def public_config(cfg: dict) -> dict:
    """The config as it is written to disk: without the builders' private keys."""
    out = json.loads(json.dumps(cfg))
    for lc in out["layers"]:
        lc.pop("_rank", None)
    return out


def write_checkpoint(path: str, cfg: dict, tensors: dict[str, torch.Tensor]) -> str:
    """config.json + model.safetensors (bfloat16): 8-byte little-endian header length, JSON header, raw data."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(public_config(cfg), f)
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return path


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(((got - ref) ** 2).mean()) / (np.sqrt((ref ** 2).mean()) + 1e-30))
