"""Zinunex as data: a pre-norm decoder whose layers choose between attention over a cached latent with a sliding window
(some of them reading the latent that an earlier layer cached) and grouped-query attention whose values are its keys and
whose softmax has a sink, every layer with a mixture of ungated experts under a scored router, and a per-layer input
from the token's id at the end of every layer.

``config.json`` (every size, and every constant that can differ between models of the design, is read from it):

* ``architecture``: "Zinunex"; ``vocab``, ``width``; ``norm.eps``; ``token_side.dim`` (absent: no per-layer input);
* ``layers``: a list; entry i has ``type`` (``latent_attention`` or ``attention``), ``mixer`` (its sizes and constants)
  and ``mlp`` (``{kind: moe, router: {experts, top, scale, groups: {count, keep}}, expert: {ff}, shared: {ff}}`` or null);
  its tensors start with ``l<i>.``.

The network: ``x = embed[token]``; per layer ``x += mixer(rms(x) * norm1)``, ``x += ff(rms(x) * norm2)``, then
``x += rms(proj(gelu_tanh(gate x) * side_embed[token, layer's columns])) * side.norm``; ``logits = head(rms(x) *
final.norm)``.

* ``latent_attention`` (``parts/latent_attention.py``): ``heads, dim, rot_dim, vdim, kv_rank, scale, mask: {size}, rot:
  {base, dims, scaling: {factor, original, fast, slow}}``, optionally ``kv_from: j``.  Queries are one projection, laid
  out per head as [dim | rot_dim]; the down-projection ``dkv`` gives the latent (RMS norm with ``dkv.norm``) and one
  rotated key part for all heads; ``uk``, ``uv`` per head.  The rotation pairs neighbours and follows the ramp law of
  ``parts/position.py`` (its magnitude multiplies cosine and sine); ``scale`` is used as given.  With ``kv_from`` the
  layer has no ``dkv``: it reads what layer j cached.
* ``attention`` (``parts/window_attention.py``): ``heads, kv_heads, dim, vdim, scale, rot: {base, dims, scaling:
  {factor}}``; projections ``q`` and ``k`` only, the values are the keys before the rotation; the rotation pairs value
  i with ``i + dims / 2``, every frequency divided by ``factor``; causal; ``sink``: a learned number per head in the
  softmax's denominator.
* the mixture (``parts/feed_forward.py``, kind ``moe_routed``): scores ``sigmoid(router h)``, the choice by score plus
  ``correction`` within the best groups, weights ``scale`` times the score; experts ``e<k>.up`` / ``e<k>.down`` with a
  squared ReLU; the shared expert times ``sigmoid(shared.sg h)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

ARCHITECTURE = "Zinunex"
# The design has no table of positions and hence no largest position of its own; this bounds what one request may hold.
MAX_POSITIONS = 1 << 17
MIXER_TYPES = ("latent_attention", "attention")


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
class RotationConfig:
    """``rot``: base, rotated dimensions, and the constants of its scaling law (which law it is follows from the
    mixer's type: a ramp for the latent attention, one factor for the other)."""

    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]      # the law's constants by name, in the file's spelling

    @classmethod
    def from_dict(cls, raw: Optional[Mapping[str, Any]], where: str, keys: Tuple[str, ...]) -> Optional["RotationConfig"]:
        if raw is None:
            return None
        scaling = _obj(raw, "scaling", where, optional=True)
        out = cls(_number(raw, "base", where), take(raw, "dims", int),
                  tuple((k, _number(scaling, k, where + "scaling.")) for k in keys) if scaling else None)
        if out.dims < 0 or out.dims % 2:
            raise ConfigError(f"invalid model config: {where}dims={out.dims} must be even and not negative")
        if not out.base > 0:
            raise ConfigError(f"invalid model config: {where}base must be positive")
        if out.scaling and any(not v > 0 for _, v in out.scaling):
            raise ConfigError(f"invalid model config: {where}scaling's constants must be positive")
        return out

    def to_dict(self) -> dict:
        out: dict = {"base": self.base, "dims": self.dims}
        if self.scaling:
            out["scaling"] = dict(self.scaling)
        return out

    def spec(self, kind: str, law: str) -> PartSpec:
        if not self.dims:
            return PartSpec("none")
        scaling = dict(self.scaling, kind=law) if self.scaling else None
        return PartSpec(kind, theta=self.base, rotary_dim=self.dims, scaling=scaling)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot: Optional[RotationConfig]
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        mask = _obj(raw, "mask", where, optional=True)
        source = raw.get("kv_from")
        if source is not None and (not isinstance(source, int) or isinstance(source, bool) or source < 0):
            raise ConfigError(f"invalid model config: {where}kv_from must name a layer, got {source!r}")
        out = cls(heads=_positive(raw, "heads", where), dim=_positive(raw, "dim", where), rot_dim=take(raw, "rot_dim", int),
                  vdim=_positive(raw, "vdim", where), kv_rank=_positive(raw, "kv_rank", where), scale=_number(raw, "scale", where),
                  window=_positive(mask, "size", where + "mask.") if mask else None,
                  rot=RotationConfig.from_dict(_obj(raw, "rot", where, optional=True), where + "rot.", ("factor", "original", "fast", "slow")),
                  kv_from=source)
        if out.rot_dim < 0:
            raise ConfigError(f"invalid model config: {where}rot_dim must not be negative")
        if out.rot and out.rot.dims > out.rot_dim:
            raise ConfigError(f"invalid model config: {where}rot.dims={out.rot.dims} exceeds rot_dim={out.rot_dim}")
        return out

    def to_dict(self) -> dict:
        out: dict = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                     "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot:
            out["rot"] = self.rot.to_dict()
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "SinkAttentionConfig":
        out = cls(heads=_positive(raw, "heads", where), kv_heads=_positive(raw, "kv_heads", where), dim=_positive(raw, "dim", where),
                  vdim=_positive(raw, "vdim", where), scale=_number(raw, "scale", where),
                  rot=RotationConfig.from_dict(_obj(raw, "rot", where, optional=True), where + "rot.", ("factor",)))
        if out.heads % out.kv_heads:
            raise ConfigError(f"invalid model config: {where}heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        if out.vdim != out.dim:
            raise ConfigError(f"invalid model config: {where}vdim={out.vdim} differs from dim={out.dim}, but the values are the keys")
        if out.rot and out.rot.dims > out.dim:
            raise ConfigError(f"invalid model config: {where}rot.dims={out.rot.dims} exceeds dim={out.dim}")
        if raw.get("mask") is not None:
            raise ConfigError(f"unsupported option: {where}mask (this mixer sees every earlier token)")
        return out

    def to_dict(self) -> dict:
        out: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot:
            out["rot"] = self.rot.to_dict()
        return out


_MIXER_CONFIGS = {"latent_attention": LatentAttentionConfig, "attention": SinkAttentionConfig}


@dataclass(frozen=True)
class MixtureConfig:
    experts: int
    top: int
    ff: int
    scale: float
    groups: int
    keep: int
    shared_ff: int                # 0: no shared expert

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MixtureConfig":
        kind = take(raw, "kind", str)
        if kind != "moe":
            raise ConfigError(f"unsupported option: {where}kind={kind!r} (moe)")
        router, expert = _obj(raw, "router", where), _obj(raw, "expert", where)
        groups = _obj(router, "groups", where + "router.", optional=True)
        shared = _obj(raw, "shared", where, optional=True)
        out = cls(experts=_positive(router, "experts", where + "router."), top=_positive(router, "top", where + "router."),
                  ff=_positive(expert, "ff", where + "expert."),
                  scale=_number(router, "scale", where + "router.") if router.get("scale") is not None else 1.0,
                  groups=_positive(groups, "count", where + "router.groups.") if groups else 1,
                  keep=_positive(groups, "keep", where + "router.groups.") if groups else 1,
                  shared_ff=_positive(shared, "ff", where + "shared.") if shared else 0)
        if out.top > out.experts:
            raise ConfigError(f"invalid model config: {where}router.top={out.top} exceeds router.experts={out.experts}")
        if out.experts % out.groups or out.keep > out.groups:
            raise ConfigError(f"invalid model config: {where}router.groups: {out.groups} groups ({out.keep} kept) of {out.experts} experts")
        if out.keep * (out.experts // out.groups) < out.top:
            raise ConfigError(f"invalid model config: {where}router: {out.keep} groups of {out.experts // out.groups} experts cannot give top={out.top}")
        return out

    def to_dict(self) -> dict:
        out: dict = {"kind": "moe", "expert": {"ff": self.ff},
                     "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                                "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class ZinunexLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[MixtureConfig]


@dataclass(frozen=True)
class ZinunexConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                 # 0: no per-layer input from the token's id
    layers: Tuple[ZinunexLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def max_model_len(self) -> int:
        return MAX_POSITIONS

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZinunexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("invalid model config: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"invalid model config: layers[{i}] must be an object")
            kind = take(entry, "type", str)
            if kind not in _MIXER_CONFIGS:
                raise ConfigError(f"unsupported option: {where}type={kind!r} (one of {', '.join(MIXER_TYPES)})")
            mlp = _obj(entry, "mlp", where, optional=True)
            layers.append(ZinunexLayerConfig(kind, _MIXER_CONFIGS[kind].from_dict(_obj(entry, "mixer", where), where + "mixer."),
                                             MixtureConfig.from_dict(mlp, where + "mlp.") if mlp else None))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if layer.type != "latent_attention" or m.kv_from is None:
                continue
            where = f"layers[{i}].mixer."
            if m.kv_from >= i or layers[m.kv_from].type != "latent_attention" or layers[m.kv_from].mixer.kv_from is not None:
                raise ConfigError(f"invalid model config: {where}kv_from={m.kv_from} must name an earlier latent_attention layer with a down-projection of its own")
            src = layers[m.kv_from].mixer
            if (src.kv_rank, src.rot_dim, src.rot) != (m.kv_rank, m.rot_dim, m.rot):
                raise ConfigError(f"invalid model config: {where}kv_rank, rot_dim and rot must equal those of layer {m.kv_from}, whose cache it reads")
        eps = _number(_obj(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError("invalid model config: norm.eps must be positive")
        side = _obj(raw, "token_side", "", optional=True)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""), norm_eps=eps,
                   side_dim=_positive(side, "dim", "token_side.") if side else 0, layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None} for l in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _mixer_spec(layer: ZinunexLayerConfig, eps: float) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        position = m.rot.spec("rope_interleaved", "ramp") if m.rot else PartSpec("none")
        return PartSpec("latent_attention", name="mix", num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=0,
                        kv_rank=m.kv_rank, scale=m.scale, eps=eps, sink=False, gate=False, window=m.window,
                        own_cache=m.kv_from is None, position=position)
    position = m.rot.spec("rope_half", "linear") if m.rot else PartSpec("none")
    return PartSpec("window_attention", name="mix", num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                    scale=m.scale, qk_norm="none", eps=eps, sink="learned", value_from_key=True, position=position,
                    names=("q", "k", "v", "o", "vmix", "q.norm", "k.norm", "sink"))


def zinunex_spec(cfg: ZinunexConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", eps=cfg.norm_eps, weight_suffix="")
    layers = []
    cache_source = {}
    for i, layer in enumerate(cfg.layers):
        mixer = _mixer_spec(layer, cfg.norm_eps)
        if layer.type == "latent_attention" and layer.mixer.kv_from is not None:
            cache_source[i] = layer.mixer.kv_from          # no layer runs twice: a layer's run has the layer's number
        f = layer.mlp
        if f is None:
            ffn = PartSpec("none", name="mlp")
        else:
            ffn = PartSpec("moe_routed", name="mlp", experts=f.experts, top=f.top, intermediate_size=f.ff, activation="relu2",
                           score="sigmoid", correction_name="correction", groups=(f.groups, f.keep), route_scale=f.scale,
                           router_name="router", expert_names=("e{}.up", "e{}.down"), shared_size=f.shared_ff,
                           shared_names=("shared.up", "shared.down"), shared_gate_name="shared.sg")
        after = None
        if cfg.side_dim:
            after = PartSpec("token_side", name="side", dim=cfg.side_dim, index=i, layers=len(cfg.layers), vocab_size=cfg.vocab,
                             eps=cfg.norm_eps, table_name="side.embed", names=("gate", "proj", "norm"))
        block = PartSpec("prenorm", norm_names=("norm1", "norm2"), after=after)
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, layers=tuple(layers),
                     final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm", lm_head_name="head",
                     cache_source=cache_source, eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture(ARCHITECTURE, ZinunexConfig.from_dict, zinunex_spec, replace=True)
