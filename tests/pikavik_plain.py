"""Plain, slow restatement of the Pikavik design in float64 on the CPU — the oracle of tests/test_pikavik_*.py.
One function per mechanism, written from the design's equations; it shares no code with ssd_b200 (it reads the raw
checkpoint tensors by name, not the packed layout, and keeps its own state dictionaries).

Notation: x residual stream, h the block's normed input, t a position, H heads.  Every mixer takes the rows of ONE
sequence (`h` [n, width], first position `p0`) and a state dict that carries what the sequence left behind, so a prompt
can be fed whole, in portions or token by token."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def block_norm(x, weight, eps):
    """RMS norm with a unit-offset weight (scale 1 + w)."""
    return unit_rms(x, eps) * (1.0 + weight)


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(scores: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """scores [E] of one token -> (chosen experts, weights).  A group's score is the sum of its two best scores."""
    E = scores.numel()
    per = E // groups
    gscore = []
    for g in range(groups):
        s = sorted(scores[g * per:(g + 1) * per].tolist(), reverse=True)
        gscore.append(sum(s[:2]))
    kept = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
    allowed = [e for g in kept for e in range(g * per, (g + 1) * per)]
    chosen = sorted(allowed, key=lambda e: (-scores[e].item(), e))[:top]
    w = torch.stack([scores[e] for e in chosen])
    return chosen, w / (w.sum() + 1e-20) * scale


def moe_ff(h, W, p, m):
    """h [n, width]; W raw tensors; p = 'l<i>.mlp'; m = the layer's mlp config."""
    r = m["router"]
    grp = r.get("groups") or {}
    groups = grp.get("count", 1)
    keep = grp.get("keep", groups)
    scores = torch.sigmoid(h @ W[p + ".router"].T)
    out = torch.zeros(h.shape[0], W[p + ".e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        chosen, wts = route(scores[t], r["top"], groups, keep, r.get("scale", 1.0))
        for e, wt in zip(chosen, wts):
            q = f"{p}.e{e}"
            out[t] += wt * clamped_expert(h[t:t + 1], W[q + ".gate"], W[q + ".up"], W[q + ".down"], m["expert"]["limit"])[0]
    sh = m.get("shared")
    if sh:
        q = p + ".shared"
        out = out + clamped_expert(h, W[q + ".gate"], W[q + ".up"], W[q + ".down"], sh["limit"]) * torch.sigmoid(h @ W[q + ".sg"].T)
    return out


def wkv_mixer(h, W, p, mx, eps, state, p0):
    H, D = mx["heads"], mx["dim"]
    S = state.get("S", torch.zeros(H, D, D, dtype=F64))
    prev = state.get("h", torch.zeros(h.shape[1], dtype=F64))
    out = []
    for t in range(h.shape[0]):
        cur = h[t]
        mix = {s: cur + (prev - cur) * W[f"{p}.mu.{s}"] for s in "rkvgw"}
        r = (W[p + ".r"] @ mix["r"]).view(H, D)
        k = (W[p + ".k"] @ mix["k"]).view(H, D)
        v = (W[p + ".v"] @ mix["v"]).view(H, D)
        gate = torch.nn.functional.silu(W[p + ".g"] @ mix["g"])
        decay = torch.exp(-torch.exp(W[p + ".w2"] @ torch.tanh(W[p + ".w1"] @ mix["w"]) + W[p + ".w0"])).view(H, D)
        o = torch.zeros(H, D, dtype=F64)
        for hd in range(H):
            kv = torch.outer(k[hd], v[hd])
            o[hd] = (S[hd] + W[p + ".u"][hd][:, None] * kv).T @ r[hd]
            S[hd] = decay[hd][:, None] * S[hd] + kv
        o = unit_rms(o, eps).reshape(-1) * W[p + ".norm"] * gate
        out.append(W[p + ".o"] @ o)
        prev = cur
    state["S"], state["h"] = S, prev
    return torch.stack(out)


def mlstm_mixer(h, W, p, mx, eps, state, p0):
    H, D, V, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    S = state.get("S", torch.zeros(H, D, V, dtype=F64))
    nrm = state.get("n", torch.zeros(H, D, dtype=F64))
    m = state.get("m", torch.zeros(H, dtype=F64))
    out = []
    for t in range(h.shape[0]):
        cur = h[t]
        q = (W[p + ".q"] @ cur).view(H, D) * D ** -0.5
        k = (W[p + ".k"] @ cur).view(H, D)
        v = (W[p + ".v"] @ cur).view(H, V)
        i_log = cap * torch.tanh((W[p + ".i"] @ cur + W[p + ".i.b"]) / cap)
        f_log = torch.nn.functional.logsigmoid(cap * torch.tanh((W[p + ".f"] @ cur + W[p + ".f.b"]) / cap))
        m_new = torch.maximum(f_log + m, i_log)
        keep_, add = torch.exp(f_log + m - m_new), torch.exp(i_log - m_new)
        o = torch.zeros(H, V, dtype=F64)
        for hd in range(H):
            S[hd] = keep_[hd] * S[hd] + add[hd] * torch.outer(k[hd], v[hd])
            nrm[hd] = keep_[hd] * nrm[hd] + add[hd] * k[hd]
            den = max(abs(float(nrm[hd] @ q[hd])), math.exp(-float(m_new[hd]))) + 1e-6
            o[hd] = (S[hd].T @ q[hd]) / den
        m = m_new
        o = unit_rms(o, eps).reshape(-1) * W[p + ".norm"] * torch.sigmoid(W[p + ".g"] @ cur)
        out.append(W[p + ".o"] @ o)
    state["S"], state["n"], state["m"] = S, nrm, m
    return torch.stack(out)


def rotate_half(vec, pos, dims, base):
    """vec [..., R]: the first `dims` entries are turned, entry i paired with i + dims/2."""
    half = dims // 2
    ang = pos * base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    a, b = vec[..., :half], vec[..., half:dims]
    return torch.cat([a * torch.cos(ang) - b * torch.sin(ang), b * torch.cos(ang) + a * torch.sin(ang), vec[..., dims:]], -1)


def latent_attention_mixer(h, W, p, mx, eps, state, p0):
    H, D, R, V, KR = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    dims, base = mx["rot"]["dims"], mx["rot"]["base"]
    lat = state.setdefault("c", [])      # one latent per cached token
    rot = state.setdefault("kr", [])     # one rotated key part per cached token
    out = []
    for t in range(h.shape[0]):
        pos = p0 + t
        cur = h[t]
        cq = unit_rms(W[p + ".dq"] @ cur, eps) * W[p + ".dq.norm"]
        q = (W[p + ".uq"] @ cq).view(H, D + R)
        down = W[p + ".dkv"] @ cur
        lat.append(unit_rms(down[:KR], eps) * W[p + ".dkv.norm"])
        rot.append(rotate_half(down[KR:], pos, dims, base))
        C, KRm = torch.stack(lat), torch.stack(rot)          # [ctx, KR], [ctx, R]
        keys = (C @ W[p + ".uk"].T).view(-1, H, D)
        vals = (C @ W[p + ".uv"].T).view(-1, H, V)
        o = torch.zeros(H, V, dtype=F64)
        for hd in range(H):
            qr = rotate_half(q[hd, D:], pos, dims, base)
            s = (keys[:, hd] @ q[hd, :D] + KRm @ qr) * mx["scale"]
            big = torch.maximum(s.max(), W[p + ".sink"][hd])
            e = torch.exp(s - big)
            o[hd] = (e[:, None] * vals[:, hd]).sum(0) / (e.sum() + torch.exp(W[p + ".sink"][hd] - big))
        out.append(W[p + ".o"] @ o.reshape(-1))
    return torch.stack(out)


MIXERS = {"wkv": wkv_mixer, "mlstm": mlstm_mixer, "latent_attention": latent_attention_mixer}


class PlainModel:
    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    def new_state(self):
        return [dict() for _ in self.cfg["layers"]]

    def run(self, tokens, state=None, p0=0, layers_out=None):
        """Logits [n, vocab] of `tokens` continuing a sequence at position p0 with `state` (None: a new sequence)."""
        cfg, W = self.cfg, self.W
        eps = cfg["norm"]["eps"]
        state = state if state is not None else self.new_state()
        x = W["embed"][torch.tensor(list(tokens))]
        for i, lc in enumerate(cfg["layers"]):
            p = f"l{i}"
            h = block_norm(x, W[p + ".norm1"], eps)
            y = MIXERS[lc["type"]](h, W, p + ".mix", lc["mixer"], eps, state[i], p0) * W[p + ".ls1"]
            if lc.get("mlp"):
                y = y + moe_ff(h, W, p + ".mlp", lc["mlp"]) * W[p + ".ls2"]
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        return block_norm(x, W["final.norm"], eps) @ W["head"].T

    def greedy(self, prompt, n_new):
        state = self.new_state()
        logits = self.run(prompt, state, 0)
        out, pos = [], len(prompt)
        for _ in range(n_new):
            tok = int(torch.argmax(logits[-1]))
            out.append(tok)
            logits = self.run([tok], state, pos)
            pos += 1
        return out
