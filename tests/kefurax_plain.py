"""Plain, slow restatement of the Kefurax design in float64 on the CPU — the oracle of tests/test_kefurax_*.py.
One function per mechanism, written from the design's equations; it shares no code with ssd_b200 (it reads the raw
checkpoint tensors by name, not the packed layout, and keeps its own state dictionaries).

Notation: x residual stream (a sublayer reads x itself; the norm sits on the sublayer's OUTPUT), t a position, H heads.
Every mixer takes the rows of ONE sequence (`h` [n, width], first position `p0`) and a state dict that carries what the
sequence left behind (recurrent matrices, the last taps - 1 inputs of every short convolution, cached keys and values),
so a prompt can be fed whole, in portions or token by token."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    """RMS norm with a plain weight."""
    return unit_rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(u, w, bias, state, key):
    """Causal per-channel convolution over time.  u [n, C]; w [C, taps], the last column multiplies the current token;
    zeros before the start of the sequence.  state[key] keeps the last taps - 1 inputs."""
    C, taps = w.shape
    hist = state.get(key)
    if hist is None:
        hist = torch.zeros(taps - 1, C, dtype=F64)
    full = torch.cat([hist, u], 0)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * full[t + j]
    if bias is not None:
        out = out + bias
    state[key] = full[full.shape[0] - (taps - 1):].clone() if taps > 1 else torch.zeros(0, C, dtype=F64)
    return out


# ------------------------------------------------------------------------------------------------ rglru
def rglru_mixer(h, W, p, mx, state):
    """Recurrent block: a gelu branch y and a convolved branch u that drives a gated diagonal recurrence."""
    width, blocks = mx["width"], mx["blocks"]
    bs = width // blocks
    y = gelu_tanh(h @ W[p + ".y"].T + W[p + ".y.b"])
    u = short_conv(h @ W[p + ".x"].T + W[p + ".x.b"], W[p + ".conv"], W[p + ".conv.b"], state, "conv")
    S = state.get("S", torch.zeros(width, dtype=F64))
    sp = softplus(W[p + ".lam"])
    out = []
    for t in range(h.shape[0]):
        r = torch.zeros(width, dtype=F64)
        i = torch.zeros(width, dtype=F64)
        for b in range(blocks):
            ub = u[t, b * bs:(b + 1) * bs]
            r[b * bs:(b + 1) * bs] = torch.sigmoid(W[p + ".ra"][b] @ ub + W[p + ".ra.b"][b])
            i[b * bs:(b + 1) * bs] = torch.sigmoid(W[p + ".ri"][b] @ ub + W[p + ".ri.b"][b])
        a = torch.exp(-8.0 * r * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * i * u[t]
        out.append(S * y[t])
    state["S"] = S
    return torch.stack(out) @ W[p + ".o"].T


# ------------------------------------------------------------------------------------------------ softmax attention
def rotary_table(rot):
    """(frequencies [dims / 2], factor on cos and sin) with the YaRN correction if rot has 'scaling'."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = sc["factor"], sc["original"]

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, pos, rot):
    """v [n, heads, dim]; pairs (2i, 2i+1) of the first rot.dims dimensions turn by pos * f_i."""
    freqs, mult = rotary_table(rot)
    dims = rot["dims"]
    ang = torch.tensor(pos, dtype=F64)[:, None] * freqs[None, :]
    cos, sin = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def sink_attention(h, W, p, mx, eps, state, p0, sink=1.0):
    """Grouped-query causal softmax attention whose denominator has one extra 1 (a sink of score 0 without a value),
    rotary positions, unit-RMS queries and keys, and a sigmoid output gate.  (`sink` is the design's 1; the tests pass 0
    to show that a plain softmax would give other numbers.)"""
    n = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = list(range(p0, p0 + n))
    q = (h @ W[p + ".q"].T).view(n, H, D)
    k = (h @ W[p + ".k"].T).view(n, G, D)
    v = (h @ W[p + ".v"].T).view(n, G, V)
    rot = mx.get("rot")
    if rot and rot.get("dims", 0) >= 2:
        q, k = rotate_interleaved(q, pos, rot), rotate_interleaved(k, pos, rot)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    K = torch.cat([state["K"], k], 0) if "K" in state else k
    Vc = torch.cat([state["V"], v], 0) if "V" in state else v
    state["K"], state["V"] = K, Vc
    out = torch.zeros(n, H, V, dtype=F64)
    for t in range(n):
        ctx = p0 + t + 1
        for hd in range(H):
            g = hd // (H // G)
            s = (K[:ctx, g] @ q[t, hd]) * mx["scale"]
            m = max(s.max().item(), 0.0)
            e = torch.exp(s - m)
            out[t, hd] = (e[:, None] * Vc[:ctx, g]).sum(0) / (sink * math.exp(-m) + e.sum())
    gate = torch.sigmoid(h @ W[p + ".g"].T)
    return (out.reshape(n, H * V) * gate) @ W[p + ".o"].T


# ------------------------------------------------------------------------------------------------ gated delta rule
def gated_delta_mixer(h, W, p, mx, eps, state):
    n = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(short_conv(h @ W[p + ".q"].T, W[p + ".q.conv"], None, state, "cq")).view(n, G, D)
    k = silu(short_conv(h @ W[p + ".k"].T, W[p + ".k.conv"], None, state, "ck")).view(n, G, D)
    v = silu(short_conv(h @ W[p + ".v"].T, W[p + ".v.conv"], None, state, "cv")).view(n, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + ".b"].T)
    decay = torch.exp(-torch.exp(W[p + ".A_log"]) * softplus(h @ W[p + ".a"].T + W[p + ".dt_bias"]))
    S = state.get("S", torch.zeros(H, D, V, dtype=F64))
    out = torch.zeros(n, H, V, dtype=F64)
    for t in range(n):
        for hd in range(H):
            g = hd // (H // G)
            Sh = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - Sh.T @ k[t, g])
            Sh = Sh + torch.outer(k[t, g], u)
            out[t, hd] = Sh.T @ q[t, g]
            S[hd] = Sh
    state["S"] = S
    o = unit_rms(out, eps) * W[p + ".norm"] * silu(h @ W[p + ".g"].T).view(n, H, V)
    return o.reshape(n, H * V) @ W[p + ".o"].T


def parallel_mixer(h, W, p, mx, eps, state, p0):
    left = sink_attention(h, W, p + ".left", mx["left"], eps, state.setdefault("left", {}), p0)
    right = gated_delta_mixer(h, W, p + ".right", mx["right"], eps, state.setdefault("right", {}))
    return mx["left_scale"] * left + mx["right_scale"] * right


# ------------------------------------------------------------------------------------------------ selective scan
def mamba1_mixer(h, W, p, mx, state):
    n = h.shape[0]
    inner, N, R = mx["inner"], mx["state"], mx["dt_rank"]
    xz = h @ W[p + ".in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(short_conv(x, W[p + ".conv"], W[p + ".conv.b"], state, "conv"))
    dbc = x @ W[p + ".x"].T
    dt = softplus(dbc[:, :R] @ W[p + ".dt"].T + W[p + ".dt.b"])
    B, Cm = dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    A = -torch.exp(W[p + ".A_log"])
    S = state.get("S", torch.zeros(inner, N, dtype=F64))
    y = torch.zeros(n, inner, dtype=F64)
    for t in range(n):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + W[p + ".D"] * x[t]
    state["S"] = S
    return (y * silu(z)) @ W[p + ".o"].T


# ------------------------------------------------------------------------------------------------ feed-forward, model
def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + ".gate"].T) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


def mixer(kind, h, W, p, mx, eps, state, p0):
    if kind == "rglru":
        return rglru_mixer(h, W, p, mx, state)
    if kind == "parallel":
        return parallel_mixer(h, W, p, mx, eps, state, p0)
    if kind == "mamba1":
        return mamba1_mixer(h, W, p, mx, state)
    raise ValueError(kind)


def forward(cfg, W, tokens, state, p0):
    """Runs `tokens` (positions p0 ..) of one sequence.  W: name -> float64 tensor.  state: dict carried between calls
    (empty for a new sequence).  Returns (logits [n, vocab], residual stream after every layer [layers, n, width])."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    taps = []
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}"
        st = state.setdefault(i, {})
        x = x + m * rms_norm(mixer(lc["type"], x, W, p + ".mix", lc["mixer"], eps, st, p0), W[p + ".norm1"], eps)
        if lc.get("mlp"):
            if lc["mlp"].get("kind", "dense") != "dense":
                raise ValueError("unknown feed-forward kind")
            x = x + m * rms_norm(dense_ff(x, W, p + ".mlp"), W[p + ".norm2"], eps)
        taps.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(taps)
