"""Desilorn, written down plainly: one slow function per mechanism, in the precision of the tensors it is given
(the tests pass float64).  Shares no code with the package.

Notation: W width, T tokens of ONE sequence at positions 0..T-1, S residual streams, H query heads, G key/value heads,
d query/key size, dv value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


# ---- residual streams ------------------------------------------------------------------------------------------------
def streams_read(xs, w_in):
    """xs [S, T, W], w_in [S] -> the sub-layer's input before its norm, [T, W]."""
    return sum(w_in[s] * xs[s] for s in range(xs.shape[0]))


def streams_write(xs, y, w_mix, w_out):
    """All streams at once from the old ones: new[t] = sum_s mix[s, t] old[s] + out[t] y."""
    S = xs.shape[0]
    return torch.stack([sum(w_mix[s, t] * xs[s] for s in range(S)) + w_out[t] * y for t in range(S)])


# ---- what the two attentions are made of ----------------------------------------------------------------------------
def distance_slopes(H: int) -> List[float]:
    return [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def rotate_half(x, positions, base: float, dims: int):
    """x [T, heads, d]; dimension i pairs with i + dims/2 for i < dims/2; the dimensions from dims on pass unchanged."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = positions.to(x.dtype) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def sees_sliding(i, j, size: Optional[int]):
    """Whether the query at position i sees the key at position j (integers or integer tensors)."""
    return (j <= i) & ((i - j < size) if size is not None else (j <= i))


def sees_chunk(i, j, size: Optional[int]):
    return (j <= i) & ((i // size == j // size) if size is not None else (j <= i))


def attend(q, k, v, scale: float, sees, size, slopes=None, sinks=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv].  ``sinks`` [H]: a score per head that joins the softmax's
    denominator and nothing else: no key, no value, no scale, no bias."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = sees(i, j, size)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if slopes is not None:
            s = s - slopes[h] * (i - j).to(q.dtype)
        s = s.masked_fill(~seen, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sinks is not None:
            m = torch.maximum(m, sinks[h])
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sinks is not None:
            den = den + torch.exp(sinks[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out.reshape(T, H * dv)


def _project(h, w: Dict[str, torch.Tensor], name: str, heads: int, size: int):
    return (h @ w[name].T + w[name + ".b"]).view(h.shape[0], heads, size)


def attention_sliding(h, w: Dict[str, torch.Tensor], m: dict):
    """The mixer 'attention': biased projections, a query temperature, a distance bias, a sliding window and a learned
    sink per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = _project(h, w, "q", H, d), _project(h, w, "k", G, d), _project(h, w, "v", G, dv)
    temp = m.get("q_temp")
    if temp:
        factor = torch.tensor([query_temperature(p, float(temp["coef"]), int(temp["every"])) for p in range(T)], dtype=h.dtype)
        q = q * factor[:, None, None]
    size = m["mask"]["size"] if m.get("mask") else None
    o = attend(q, k, v, float(m["scale"]), sees_sliding, size, slopes=distance_slopes(H), sinks=w["sink"])
    return o @ w["o"].T


def attention_chunked(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """The mixer 'attention_2': biased projections, a norm of every query and key head with one gain for all heads,
    rotation of the first dimensions, a mask of chunks and a sink of score zero."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = _project(h, w, "q", H, d), _project(h, w, "k", G, d), _project(h, w, "v", G, dv)
    q = rms(q, eps) * w["q.norm"]
    k = rms(k, eps) * w["k.norm"]
    rot = m.get("rot")
    if rot and rot.get("dims", 0):
        pos = torch.arange(T)
        q = rotate_half(q, pos, float(rot["base"]), int(rot["dims"]))
        k = rotate_half(k, pos, float(rot["base"]), int(rot["dims"]))
    size = m["mask"]["size"] if m.get("mask") else None
    o = attend(q, k, v, float(m["scale"]), sees_chunk, size, sinks=torch.zeros(H, dtype=h.dtype))
    return o @ w["o"].T


def feed_forward(h, w: Dict[str, torch.Tensor]):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# ---- the model ---------------------------------------------------------------------------------------------------------
def run_order(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, taps: Optional[list] = None):
    """Logits [T, vocab] of one sequence fed whole.  ``taps``: a list that gets the sum of the streams after every
    layer run."""
    eps = float(config["norm"]["eps"])
    S = int(config.get("streams", 0))              # 0: one residual row and a plain sum
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = torch.stack([x] * max(S, 1))

    def sublayer(xs, p, q, fn):
        if not S:
            return xs + fn(norm_one_plus(xs[0], weights[p + f"norm{q}"], eps))[None]
        u = streams_read(xs, weights[p + f"hc{q}.in"])
        y = fn(norm_one_plus(u, weights[p + f"norm{q}"], eps))
        return streams_write(xs, y, weights[p + f"hc{q}.mix"], weights[p + f"hc{q}.out"])

    for i in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if layer["type"] == "attention":
            xs = sublayer(xs, p, 1, lambda h: attention_sliding(h, sub(weights, p + "mix."), layer["mixer"]))
        elif layer["type"] == "attention_2":
            xs = sublayer(xs, p, 1, lambda h: attention_chunked(h, sub(weights, p + "mix."), layer["mixer"], eps))
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            xs = sublayer(xs, p, 2, lambda h: feed_forward(h, sub(weights, p + "mlp.")))
        if taps is not None:
            taps.append(xs.sum(0))
    x = norm_one_plus(xs.sum(0), weights["final.norm"], eps)
    return x @ weights["embed"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt, steps: int) -> List[int]:
    """Greedy continuation, recomputing the whole sequence every step (the lower id wins a tie)."""
    toks = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(config, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


# ---- random weights for the tests ------------------------------------------------------------------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Name -> shape of every tensor a model of this configuration has."""
    W, V, S = config["width"], config["vocab"], int(config.get("streams", 0))
    out: Dict[str, tuple] = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            out[p + f"mix.{name}"] = (rows, W)
            out[p + f"mix.{name}.b"] = (rows,)
        out[p + "mix.o"] = (W, H * dv)
        if layer["type"] == "attention":
            out[p + "mix.sink"] = (H,)
        else:
            out[p + "mix.q.norm"] = (d,)
            out[p + "mix.k.norm"] = (d,)
        subs = ["hc1"]
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out[p + "norm2"] = (W,)
            out[p + "mlp.gate"] = (ff, W)
            out[p + "mlp.up"] = (ff, W)
            out[p + "mlp.down"] = (W, ff)
            subs.append("hc2")
        if S:
            for q in subs:
                out[p + f"{q}.in"] = (S,)
                out[p + f"{q}.out"] = (S,)
                out[p + f"{q}.mix"] = (S, S)
    return out


def random_model(config: dict, seed: int, sharp: float = 2.5, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights whose values are bfloat16 numbers.  ``sharp`` scales the query projections, so that the scores spread out
    and a wrong, missing or stale key moves the logits."""
    g = torch.Generator().manual_seed(seed)
    t: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if len(shape) == 2 and not leaf.endswith(".mix") or leaf in ("mix.o",):
            x = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf == "mix.q":
                x = x * sharp
            if name == "embed":
                x = torch.randn(shape, generator=g)
        elif leaf.endswith(".mix") and len(shape) == 2:              # stream to stream: around the identity
            x = torch.eye(shape[0]) + 0.25 * torch.randn(shape, generator=g)
        elif leaf.endswith(".in"):
            x = 1.0 / shape[0] + 0.3 * torch.randn(shape, generator=g)
        elif leaf.endswith(".out"):
            x = 1.0 + 0.4 * torch.randn(shape, generator=g)
        elif leaf in ("mix.q.norm", "mix.k.norm"):
            x = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf == "mix.sink":
            x = 1.5 * torch.randn(shape, generator=g)
        elif leaf.endswith(".b"):
            x = 0.3 * torch.randn(shape, generator=g)
        else:                                                        # norm weights, stored around zero
            x = 0.2 * torch.randn(shape, generator=g)
        t[name] = x.bfloat16().to(dtype)
    return t
