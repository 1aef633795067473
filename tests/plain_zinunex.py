"""Zinunex, written down plainly: one slow function per mechanism, in the precision of the tensors it is given (the
tests pass float64 or float32).  Shares no code with the package.

Notation: W width, T tokens of ONE sequence at positions 0..T-1, H query heads, G key/value heads, d query/key size,
dr rotated part, dv value size, rk latent size, E experts.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---- rotations ---------------------------------------------------------------------------------------------------------
def plain_frequencies(base: float, dims: int) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def linear_frequencies(base: float, dims: int, factor: float) -> List[float]:
    """Every frequency divided by one factor."""
    return [f / factor for f in plain_frequencies(base, dims)]


def ramp_frequencies(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """Frequencies blended between f and f / factor along a ramp over the pair index, and the number both cosine and
    sine are multiplied by."""
    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, layout: str, magnitude: float = 1.0):
    """x [T, heads, n]: the first 2 * len(freqs) values of every head are rotated, pair i = (2i, 2i+1) for
    ``neighbours`` or (i, i + len(freqs)) for ``halves``; the rest pass unchanged."""
    out = x.clone()
    n = len(freqs)
    for i, f in enumerate(freqs):
        a = positions.to(x.dtype) * f
        c, s = (torch.cos(a) * magnitude)[:, None], (torch.sin(a) * magnitude)[:, None]
        e0, e1 = (2 * i, 2 * i + 1) if layout == "neighbours" else (i, i + n)
        u, v = x[..., e0], x[..., e1]
        out[..., e0] = u * c - v * s
        out[..., e1] = v * c + u * s
    return out


def rotation_of(rot: Optional[dict], kind: str):
    """(frequencies, magnitude) of a mixer's ``rot`` entry; ``kind`` says which scaling law its ``scaling`` follows."""
    if not rot or not rot.get("dims"):
        return [], 1.0
    base, dims, sc = float(rot["base"]), int(rot["dims"]), rot.get("scaling")
    if not sc:
        return plain_frequencies(base, dims), 1.0
    if kind == "ramp":
        return ramp_frequencies(base, dims, float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    return linear_frequencies(base, dims, float(sc["factor"])), 1.0


# ---- softmax over visible keys, with or without a sink ---------------------------------------------------------------------
def masked_softmax(scores, seen, sink=None):
    """scores [T, T]; seen: boolean table; sink: a number whose exponential joins the denominator only."""
    s = scores.masked_fill(~seen, -math.inf)
    if sink is None:
        return torch.softmax(s, -1)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.reshape(1, 1).to(s.dtype))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink.to(s.dtype) - m))


def sees(T: int, window: Optional[int]):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) if window is None else (j <= i) & (i - j < window)


# ---- the two mixers ------------------------------------------------------------------------------------------------------
def latent_parts(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """What a latent layer leaves for itself and for the layers that read it: (latent c [T, rk], rotated shared key
    part [T, dr])."""
    T = h.shape[0]
    rk, dr = m["kv_rank"], m["rot_dim"]
    down = h @ w["dkv"].T
    c = rms(down[:, :rk], eps) * w["dkv.norm"]
    freqs, mag = rotation_of(m.get("rot"), "ramp")
    kr = rotate(down[:, rk:].reshape(T, 1, dr), torch.arange(T), freqs, "neighbours", mag).reshape(T, dr)
    return c, kr


def latent_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float, kept=None):
    """h [T, W] -> (output [T, W], (c, kr)).  ``kept``: another layer's (c, kr) to use instead of own ones."""
    T = h.shape[0]
    H, d, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kept if kept is not None else latent_parts(h, w, m, eps)
    q = (h @ w["q"].T).view(T, H, d + dr)
    freqs, mag = rotation_of(m.get("rot"), "ramp")
    q_rot = rotate(q[..., d:], torch.arange(T), freqs, "neighbours", mag)
    k = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    mask = m.get("mask")
    seen = sees(T, int(mask["size"]) if mask else None)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        s = (q[:, hh, :d] @ k[:, hh].T + q_rot[:, hh] @ kr.T) * float(m["scale"])
        out[:, hh] = masked_softmax(s, seen) @ v[:, hh]
    return out.reshape(T, H * dv) @ w["o"].T, (c, kr)


def sink_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Grouped-query attention over every earlier token whose values are the keys as projected; a learned number per
    head joins the softmax's denominator."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = k
    freqs, mag = rotation_of(m.get("rot"), "linear")
    pos = torch.arange(T)
    q, k = rotate(q, pos, freqs, "halves", mag), rotate(k, pos, freqs, "halves", mag)
    seen = sees(T, None)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        out[:, hh] = masked_softmax(s, seen, w["sink"][hh]) @ v[:, g]
    return out.reshape(T, H * d) @ w["o"].T


# ---- feed-forward ------------------------------------------------------------------------------------------------------
def choose_experts(z, correction, top: int, groups: int, keep: int):
    """z [E] router logits -> (indices of the chosen experts, their scores without the correction)."""
    E = z.shape[0]
    s = torch.sigmoid(z)
    c = s + correction
    size = E // groups
    marks = []
    for g in range(groups):
        part = torch.sort(c[g * size:(g + 1) * size], descending=True).values
        marks.append(float(part[:2].sum()))
    best = sorted(range(groups), key=lambda g: (-marks[g], g))[:keep]
    allowed = torch.full((E,), -math.inf, dtype=z.dtype)
    for g in best:
        allowed[g * size:(g + 1) * size] = c[g * size:(g + 1) * size]
    order = sorted(range(E), key=lambda e: (-float(allowed[e]), e))[:top]
    return order, [s[e] for e in order]


def expert(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def mixture(h, w: Dict[str, torch.Tensor], f: dict, routers: Optional[list] = None):
    """h [T, W] -> [T, W]."""
    r = f["router"]
    E, top, scale = int(r["experts"]), int(r["top"]), float(r.get("scale", 1.0))
    gr = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ w["router"].T
    if routers is not None:
        routers.append((f, z, w["correction"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, scores = choose_experts(z[t], w["correction"].to(z.dtype), top, int(gr["count"]), int(gr["keep"]))
        for e, s in zip(chosen, scores):
            out[t] += s * scale * expert(h[t], w[f"e{e}.up"], w[f"e{e}.down"])
    if f.get("shared"):
        gate = torch.sigmoid(h @ w["shared.sg"].T)                       # [T, 1]
        out = out + gate * expert(h, w["shared.up"], w["shared.down"])
    return out


# ---- the model -----------------------------------------------------------------------------------------------------------
def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, tap: Optional[Callable] = None,
            routers: Optional[list] = None):
    """Logits [T, vocab] of one sequence fed whole; ``tap(layer, x)`` sees the stream after every layer."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(config["norm"]["eps"])
    x = weights["embed"][ids]
    side = config.get("token_side")
    kept: Dict[int, tuple] = {}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = rms(x, eps) * weights[p + "norm1"]
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            y, kept[i] = latent_mixer(h, sub(weights, p + "mix."), m, eps, kept[src] if src is not None else None)
        else:
            y = sink_mixer(h, sub(weights, p + "mix."), m, eps)
        x = x + y
        if L.get("mlp"):
            h = rms(x, eps) * weights[p + "norm2"]
            x = x + mixture(h, sub(weights, p + "mlp."), L["mlp"], routers)
        if side:
            n = int(side["dim"])
            e = weights["side.embed"][ids][:, i * n:(i + 1) * n]
            y = (gelu_tanh(x @ weights[p + "side.gate"].T) * e) @ weights[p + "side.proj"].T
            x = x + rms(y, eps) * weights[p + "side.norm"]
        if tap is not None:
            tap(i, x)
    return (rms(x, eps) * weights["final.norm"]) @ weights["head"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: List[int], steps: int) -> List[int]:
    seq = list(prompt)
    for _ in range(steps):
        seq.append(int(forward(config, weights, seq)[-1].argmax()))
    return seq[len(prompt):]


# ---- how safe the routers' choices are ------------------------------------------------------------------------------------
def choice_margins(z, correction, top: int, groups: int, keep: int):
    """For rows of router logits z [N, E]: the smallest amount by which a choice score (or half a group's mark) would
    have to move to change which groups are kept or which experts are chosen, per row [N]."""
    N, E = z.shape
    c = torch.sigmoid(z) + correction
    size = E // groups
    margin = torch.full((N,), math.inf, dtype=z.dtype)
    allowed = torch.ones(N, E, dtype=torch.bool)
    if groups > 1:
        marks = c.view(N, groups, size).topk(min(2, size), dim=-1).values.sum(-1)
        ranked = marks.sort(-1, descending=True)
        if keep < groups:
            margin = torch.minimum(margin, (ranked.values[:, keep - 1] - ranked.values[:, keep]) / 2)
        kept = torch.zeros(N, groups, dtype=torch.bool)
        kept.scatter_(1, ranked.indices[:, :keep], True)
        allowed = kept.repeat_interleave(size, dim=1)
    ranked = c.masked_fill(~allowed, -math.inf).sort(-1, descending=True).values
    if top < keep * size:
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    return margin


def router_margin(config: dict, weights: Dict[str, torch.Tensor], tokens) -> float:
    """The smallest margin (see ``choice_margins``) over the sequence's tokens and layers; the tests assert that their
    weights leave a safe one, so that an engine that rounds differently still chooses the same experts."""
    seen: list = []
    forward(config, weights, tokens, routers=seen)
    worst = math.inf
    for f, z, correction in seen:
        r = f["router"]
        gr = r.get("groups") or {"count": 1, "keep": 1}
        worst = min(worst, float(choice_margins(z, correction.to(z.dtype), int(r["top"]), int(gr["count"]), int(gr["keep"])).min()))
    return worst


# ---- random weights for the tests -------------------------------------------------------------------------------------------
def random_model(config: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights whose values are bfloat16 numbers.  The routers are made robust against rounding, so that a bfloat16
    engine and this implementation choose the same experts: the first E columns of the embedding carry, per token id, the
    router's logits (a router's row e reads column e, plus a little of everything else), drawn again until every layer's
    choice has a safe margin at every size the stream's norm may have; every tensor that writes into the stream is small
    in those columns."""
    g = torch.Generator().manual_seed(seed)
    W, V = config["width"], config["vocab"]
    mixtures = [(i, L["mlp"]) for i, L in enumerate(config["layers"]) if L.get("mlp")]
    E_max = max([f["router"]["experts"] for _, f in mixtures] + [0])
    assert E_max < W

    def mat(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).bfloat16().to(dtype)

    def vec(n, around=0.0, spread=0.1):
        return (around + spread * torch.randn(n, generator=g)).bfloat16().to(dtype)

    def writer(i, gain=0.4):                         # [W, i]: output rows of the router's columns are small
        m = torch.randn(W, i, generator=g) * gain / math.sqrt(i)
        m[:E_max] *= 0.003
        return m.bfloat16().to(dtype)

    t: Dict[str, torch.Tensor] = {"head": mat(V, W, 2.0), "final.norm": vec(W, 1.0)}
    corrections = {}
    for i, f in mixtures:
        E = f["router"]["experts"]
        corrections[i] = (0.25 * torch.randn(E, generator=g)).bfloat16().double()
        t[f"l{i}.mlp.correction"] = corrections[i].to(dtype)
    embed = torch.randn(V, W, generator=g)
    if E_max:
        todo = torch.arange(V)
        for _ in range(2000):
            if not len(todo):
                break
            cand = ((torch.rand(len(todo), E_max, generator=g) * 2 - 1) * 1.3).bfloat16().double()
            ok = torch.ones(len(todo), dtype=torch.bool)
            for i, f in mixtures:
                r = f["router"]
                gr = r.get("groups") or {"count": 1, "keep": 1}
                for step in range(13):                            # logits = 2 * column / rms(stream): 0.6 to 2.7
                    lam = 0.6 * 2.0 ** (step * 0.18)
                    ok &= choice_margins(cand[:, :r["experts"]] * lam, corrections[i], r["top"], gr["count"], gr["keep"]) > 0.05
            embed[todo[ok], :E_max] = cand[ok].float()
            todo = todo[~ok]
        assert not len(todo), "no safe logits found for some token ids"
    t["embed"] = embed.bfloat16().to(dtype)
    side = config.get("token_side")
    if side:
        t["side.embed"] = torch.randn(V, len(config["layers"]) * side["dim"], generator=g).bfloat16().to(dtype)
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        t[p + "norm1"] = vec(W, 1.0)
        if L["type"] == "latent_attention":
            H, d, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "mix.q"] = mat(H * (d + dr), W, 2.0)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(rk + dr, W, 1.5), vec(rk, 1.0)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * d, rk, 1.5), mat(H * dv, rk)
            t[p + "mix.o"] = writer(H * dv)
        else:
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, W, 2.0), mat(G * d, W, 1.5)
            t[p + "mix.sink"] = vec(H, 0.0, 1.0)
            t[p + "mix.o"] = writer(H * d)
        f = L.get("mlp")
        if f:
            t[p + "norm2"] = vec(W, 1.0)
            t[p + "norm2"][:E_max] = 1.0
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(ff, W, 1.5), writer(ff)
            router = torch.randn(E, W, generator=g) * 0.02 / math.sqrt(W)
            router[:, :E_max] = 0.0
            for e in range(E):
                router[e, e] = 2.0
            t[p + "mlp.router"] = router.bfloat16().to(dtype)
            if f.get("shared"):
                t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = mat(f["shared"]["ff"], W, 1.5), writer(f["shared"]["ff"])
                t[p + "mlp.shared.sg"] = mat(1, W, 2.0)
        if side:
            t[p + "side.gate"], t[p + "side.proj"] = mat(side["dim"], W), mat(W, side["dim"])
            gain = 0.3 + 0.05 * torch.randn(W, generator=g)
            gain[:E_max] = 0.003
            t[p + "side.norm"] = gain.bfloat16().to(dtype)
    return t
