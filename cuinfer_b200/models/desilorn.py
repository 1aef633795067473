"""Desilorn as data: a pre-norm decoder whose residual is several streams joined by learned coefficients
(hyper-connections), whose layers choose between two kinds of attention, and which may run a span of its layers several
times.

``config.json`` (every size, and every constant that can differ between models of the design, is read from it):

* ``architecture``: "Desilorn"; ``vocab``, ``width``; ``norm.eps``; ``streams`` (absent: one residual row per token and
  a plain residual sum);
* ``layers``: a list; entry i has ``type`` (``attention`` or ``attention_2``), ``mixer`` (its sizes) and ``mlp``
  (``{kind: dense, ff}`` or null); its tensors start with ``l<i>.``;
* ``loop``: ``{start, stop, times}`` — layers start..stop-1 run ``times`` times in a row with the same weights, every
  pass with a cache of its own; absent: every layer runs once.

The network: ``x_s = embed[token]`` for every stream s; per sub-layer q (mixer, then feed-forward) with the coefficients
``hc<q>.in`` [S], ``hc<q>.out`` [S], ``hc<q>.mix`` [S, S]: ``u = sum_s in[s] x_s``, ``y = sublayer(rms(u) (1 + norm<q>))``,
``x_t <- sum_s mix[s, t] x_s + out[t] y``; ``logits = embed (rms(sum_s x_s) (1 + final.norm))``.  Both mixers are
``parts/window_attention.py`` with biased projections (``heads, kv_heads, dim, vdim, scale, mask: {size}``):

* ``attention``: no rotation; a query temperature (``q_temp: {coef, every}``); a distance bias with the slopes
  ``2 ** (-8 (h + 1) / heads)``; a sliding window; a learned sink per head in the softmax's denominator;
* ``attention_2``: a norm of every query and key head with one gain for all heads, before the rotation; rotation in
  halves (``rot: {base, dims}``); a mask of chunks counted from position 0; one added to the softmax's denominator.

The feed-forward is ``down(gelu_tanh(gate h) * (up h))``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

ARCHITECTURE = "Desilorn"
# The design has no table of positions and hence no largest position of its own; this bounds what one request may hold.
MAX_POSITIONS = 1 << 17
MIXER_TYPES = ("attention", "attention_2")
# The distance bias of head h is 2 ** (-DISTANCE_BIAS_EXPONENT * (h + 1) / heads) per token of distance.
DISTANCE_BIAS_EXPONENT = 8.0
MAX_STREAMS = 16


def _obj(raw: Mapping[str, Any], key: str, where: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    value = raw.get(key)
    if value is None:
        if optional:
            return None
        raise ConfigError(f"invalid model config: {where}'{key}' is missing")
    if not isinstance(value, dict):
        raise ConfigError(f"invalid model config: {where}'{key}' must be an object")
    return value


def _positive(raw: Mapping[str, Any], key: str, where: str) -> int:
    try:
        v = take(raw, key, int)
    except ConfigError as exc:
        raise ConfigError(f"{exc} (in {where})") from None
    if v <= 0:
        raise ConfigError(f"invalid model config: {where}'{key}' must be positive, got {v}")
    return v


def _number(raw: Mapping[str, Any], key: str, where: str) -> float:
    try:
        return float(take(raw, key, float))
    except ConfigError as exc:
        raise ConfigError(f"{exc} (in {where})") from None


@dataclass(frozen=True)
class AttentionConfig:
    """One attention layer's sizes and constants; ``type`` says which of the two mixers reads them."""

    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                  # mask.size: the sliding window's length, or the chunk's
    temp_coef: float = 0.0                 # attention: the query temperature (every == 0: none)
    temp_every: int = 0
    rot_base: float = 1.0                  # attention_2: the rotation (dims == 0: none)
    rot_dims: int = 0

    @classmethod
    def from_dict(cls, kind: str, raw: Mapping[str, Any], where: str) -> "AttentionConfig":
        mask = _obj(raw, "mask", where, optional=True)
        fields = dict(type=kind, heads=_positive(raw, "heads", where), kv_heads=_positive(raw, "kv_heads", where),
                      dim=_positive(raw, "dim", where), vdim=_positive(raw, "vdim", where), scale=_number(raw, "scale", where),
                      window=_positive(mask, "size", where + "mask.") if mask else None)
        if kind == "attention":
            temp = _obj(raw, "q_temp", where, optional=True)
            if temp:
                fields.update(temp_coef=_number(temp, "coef", where + "q_temp."), temp_every=_positive(temp, "every", where + "q_temp."))
            if raw.get("rot") is not None:
                raise ConfigError(f"unsupported option: {where}rot (a layer of type 'attention' has no rotation)")
        else:
            rot = _obj(raw, "rot", where, optional=True)
            if rot:
                fields.update(rot_base=_number(rot, "base", where + "rot."), rot_dims=take(rot, "dims", int))
            if raw.get("q_temp") is not None:
                raise ConfigError(f"unsupported option: {where}q_temp (a layer of type 'attention_2' has no query temperature)")
        out = cls(**fields)
        if out.heads % out.kv_heads:
            raise ConfigError(f"invalid model config: {where}heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"invalid model config: {where}rot.dims={out.rot_dims} must be even and at most dim={out.dim}")
        if out.rot_dims and not out.rot_base > 0:
            raise ConfigError(f"invalid model config: {where}rot.base must be positive")
        return out

    def to_dict(self) -> dict:
        out: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.temp_every:
            out["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return out


@dataclass(frozen=True)
class DesilornLayerConfig:
    type: str
    mixer: AttentionConfig
    ff: int                       # 0: the layer has no feed-forward


@dataclass(frozen=True)
class DesilornConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int                  # 0: one residual row per token, a plain residual sum
    layers: Tuple[DesilornLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def max_model_len(self) -> int:
        return MAX_POSITIONS

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DesilornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("invalid model config: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"invalid model config: layers[{i}] must be an object")
            kind = take(entry, "type", str)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"unsupported option: {where}type={kind!r} (one of {', '.join(MIXER_TYPES)})")
            mlp = _obj(entry, "mlp", where, optional=True)
            ff = 0
            if mlp:
                if take(mlp, "kind", str) != "dense":
                    raise ConfigError(f"unsupported option: {where}mlp.kind={mlp['kind']!r} (dense)")
                ff = _positive(mlp, "ff", where + "mlp.")
            layers.append(DesilornLayerConfig(kind, AttentionConfig.from_dict(kind, _obj(entry, "mixer", where), where + "mixer."), ff))
        eps = _number(_obj(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError("invalid model config: norm.eps must be positive")
        streams = 0
        if raw.get("streams") is not None:
            streams = _positive(raw, "streams", "")
            if streams > MAX_STREAMS:
                raise ConfigError(f"unsupported option: streams={streams} (at most {MAX_STREAMS})")
        loop = _obj(raw, "loop", "", optional=True)
        start, stop, times = (take(loop, "start", int), take(loop, "stop", int), take(loop, "times", int)) if loop else (0, 0, 1)
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ConfigError(f"invalid model config: loop start={start} stop={stop} times={times} does not fit {len(layers)} layers")
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""), norm_eps=eps, streams=streams,
                   layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None}
                          for l in self.layers]}
        if self.streams:
            out["streams"] = self.streams
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def run_order(cfg: DesilornConfig) -> Tuple[int, ...]:
    """Layer indices in the order they run: the looped span ``times`` times in a row, every pass a run of its own."""
    span = tuple(range(cfg.loop_start, cfg.loop_stop))
    return tuple(range(cfg.loop_start)) + span * cfg.loop_times + tuple(range(cfg.loop_stop, len(cfg.layers)))


def _mixer_spec(m: AttentionConfig, eps: float) -> PartSpec:
    common = dict(name="mix", num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
                  window=m.window, eps=eps, bias=True, bias_suffix=".b",
                  names=("q", "k", "v", "o", "vmix", "q.norm", "k.norm", "sink"))
    if m.type == "attention":
        return PartSpec("window_attention", qk_norm="none", q_temp=(m.temp_coef, m.temp_every) if m.temp_every else None,
                        distance_bias=DISTANCE_BIAS_EXPONENT, sink="learned", position=PartSpec("none"), **common)
    position = PartSpec("rope_half", theta=m.rot_base, rotary_dim=m.rot_dims) if m.rot_dims else PartSpec("none")
    return PartSpec("window_attention", qk_norm="gain", norm_first=True, chunked=True, sink="zero", position=position, **common)


def desilorn_spec(cfg: DesilornConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", eps=cfg.norm_eps, weight_suffix="", one_plus=True)
    if cfg.streams:
        block = PartSpec("hyper_prenorm", streams=cfg.streams, norm_names=("norm1", "norm2"), connection_names=("hc1", "hc2"),
                         coefficient_names=("in", "out", "mix"))
    else:
        block = PartSpec("prenorm", norm_names=("norm1", "norm2"))
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.ff:
            ffn = PartSpec("gated", name="mlp", intermediate_size=layer.ff, activation="gelu_tanh", names=("gate", "up", "down"))
        else:
            ffn = PartSpec("none", name="mlp")
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer_spec(layer.mixer, cfg.norm_eps), feed_forward=ffn, norm=norm))
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, layers=tuple(layers),
                     final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm", lm_head_name=None,
                     order=run_order(cfg), eos_token_ids=tuple(cfg.eos_token_ids), residual_streams=cfg.streams)


register_architecture(ARCHITECTURE, DesilornConfig.from_dict, desilorn_spec, replace=True)
