"""Mugulorn: a decoder-only model whose layers are listed one by one in config.json, each a pre-norm layer whose
mixer is either attention through a cached latent (sliding window, learned sink, output gate, YaRN-stretched rotary
part; a layer may read the cache of an earlier one) or a gated linear recurrence behind a short convolution, and
whose feed-forward (GELU-gated) may be absent.  Every sub-block enters the residual times ``residual_mult``.

config.json:  ``architecture`` "Mugulorn"; ``vocab``, ``width``, ``residual_mult``; ``embedding.scale``; ``norm.eps``;
``layers``: entries with ``type`` ("latent_attention" | "rglru"), ``mixer`` and ``mlp`` ({kind "dense", ff} or null).
  latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask {size} (absent: no window),
      rot {base, dims, scaling {factor, original, fast, slow} (absent: none)}, kv_from (absent: a cache of its own)
  rglru mixer: width, blocks, conv (taps)

Tensors: ``embed`` (also the output matrix), ``final.norm``, per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mlp.{gate,up,down}``, and
  latent_attention: ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}`` (no dkv, dkv.norm with kv_from)
  rglru:            ``l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}``
Matrices are [out, in].

  x = embed[token] * scale
  per layer:  x += m * mixer(rmsnorm(x; norm1));   x += m * mlp(rmsnorm(x; norm2))   (if it has one)
  logits = embed rmsnorm(x; final.norm)
The mixers' formulas stand in parts/latent_attention.py and parts/rglru.py, the feed-forward's in parts/mlp.py
(gated_gelu), the layer's in parts/block.py (prenorm_scaled), the rotation's in parts/rope.py (rope_yarn).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, cfg_get, cfg_positive
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import register_architecture

# Nothing in the design bounds a position (angles are computed from the position itself); a request's length is
# bounded by the engine's max_model_len, which defaults to this many tokens.
_DEFAULT_MAX_LEN = 32768
_MAX_POSITION = 1 << 24        # positions are exact in 32-bit floats up to here

# The constant in the exponent of the recurrence's decay, a = exp(-c r softplus(lam)): fixed by the design.
_RGLRU_DECAY = 8.0


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, original, fast, slow
    kv_from: Optional[int]


@dataclass(frozen=True)
class RecurrentMixer:
    width: int
    blocks: int
    taps: int


@dataclass(frozen=True)
class MugulornLayer:
    type: str
    mixer: Any                       # LatentMixer | RecurrentMixer
    ff: Optional[int]                # None: no feed-forward


def _obj(d: Mapping, key: str, where: str) -> Mapping:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _number(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _count(d: Mapping, key: str, where: str, least: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {where}'{key}' must be an int >= {least}, got {v!r}")
    return v


def _latent(m: Mapping, w: str, i: int, n_layers: int) -> LatentMixer:
    rot = _obj(m, "rot", w)
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"config.json: {w}rot.scaling must be an object or null")
        ws = w + "rot.scaling."
        scaling = tuple(_number(scaling, k, ws) for k in ("factor", "original", "fast", "slow"))
        if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
            raise ConfigError(f"config.json: {ws}factor, original, fast and slow must be positive")
    mask = m.get("mask")
    window = None
    if mask is not None:
        window = _count(_obj(m, "mask", w), "size", w + "mask.")
    kv_from = m.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < n_layers
                                or kv_from == i):
        raise ConfigError(f"config.json: {w}kv_from = {kv_from!r} names no other layer")
    out = LatentMixer(
        heads=_count(m, "heads", w), dim=_count(m, "dim", w), rot_dim=_count(m, "rot_dim", w, 0),
        vdim=_count(m, "vdim", w), q_rank=_count(m, "q_rank", w), kv_rank=_count(m, "kv_rank", w),
        scale=_number(m, "scale", w), window=window, rot_base=_number(rot, "base", w + "rot."),
        rot_dims=_count(rot, "dims", w + "rot.", 0), rot_scaling=scaling, kv_from=kv_from)
    if out.rot_dims % 2 or out.rot_dims > out.rot_dim:
        raise ConfigError(f"config.json: {w}rot.dims ({out.rot_dims}) must be even and at most rot_dim ({out.rot_dim})")
    if out.rot_base <= 1.0:
        raise ConfigError(f"config.json: {w}rot.base must exceed 1, got {out.rot_base}")
    return out


@dataclass(frozen=True)
class MugulornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    layers: Tuple[MugulornLayer, ...] = ()

    ARCHITECTURE: ClassVar[str] = "Mugulorn"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MugulornConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = e.get("type")
            m = _obj(e, "mixer", w)
            if kind == "latent_attention":
                mixer = _latent(m, w + "mixer.", i, len(entries))
            elif kind == "rglru":
                mixer = RecurrentMixer(width=_count(m, "width", w + "mixer."), blocks=_count(m, "blocks", w + "mixer."),
                                       taps=_count(m, "conv", w + "mixer."))
                if mixer.width % mixer.blocks:
                    raise ConfigError(f"config.json: {w}mixer.width ({mixer.width}) must be a multiple of blocks "
                                      f"({mixer.blocks})")
            else:
                raise ConfigError(f"config.json: {w}type {kind!r} is not supported (latent_attention, rglru)")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {w}mlp.kind must be 'dense' (or mlp null)")
                ff = _count(mlp, "ff", w + "mlp.")
            layers.append(MugulornLayer(kind, mixer, ff))
        for i, L in enumerate(layers):
            if L.type == "latent_attention" and L.mixer.kv_from is not None:
                j = L.mixer.kv_from
                o = layers[j]
                if j > i or o.type != "latent_attention" or o.mixer.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j}: not an earlier attention layer "
                                      "with a cache of its own")
                a, b = L.mixer, o.mixer
                if (a.kv_rank, a.rot_dim, a.rot_base, a.rot_dims, a.rot_scaling) != \
                        (b.kv_rank, b.rot_dim, b.rot_base, b.rot_dims, b.rot_scaling):
                    raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s cache but has another kv_rank, "
                                      "rot_dim or rotation")
        eps = _number(_obj(d, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        return cls(
            architecture=cls.ARCHITECTURE,
            vocab=cfg_positive("vocab", cfg_get(d, "vocab", int)),
            width=cfg_positive("width", cfg_get(d, "width", int)),
            embedding_scale=_number(_obj(d, "embedding", ""), "scale", "embedding."),
            norm_eps=eps,
            residual_mult=_number(d, "residual_mult", ""),
            layers=tuple(layers),
        )

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
                               "norm": {"eps": self.norm_eps}, "layers": []}
        for L in self.layers:
            m = L.mixer
            if L.type == "latent_attention":
                rot: Dict[str, Any] = {"base": m.rot_base, "dims": m.rot_dims}
                if m.rot_scaling is not None:
                    rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot_scaling))
                mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                                         "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"width": m.width, "blocks": m.blocks, "conv": m.taps}
            out["layers"].append({"type": L.type, "mixer": mixer,
                                  "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}})
        return out


def build_mugulorn_spec(cfg: MugulornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    # the window a cache has to keep: the widest of its owner's and its readers' (None: every row)
    keep: Dict[int, Optional[int]] = {}
    for i, L in enumerate(cfg.layers):
        if L.type != "latent_attention":
            continue
        owner = i if L.mixer.kv_from is None else L.mixer.kv_from
        w = L.mixer.window
        if owner not in keep:
            keep[owner] = w
        elif keep[owner] is not None:
            keep[owner] = None if w is None else max(keep[owner], w)
    layers, order = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        m = L.mixer
        if L.type == "latent_attention":
            own = m.kv_from is None
            owner = i if own else m.kv_from
            scaling = None if m.rot_scaling is None else dict(zip(("factor", "original", "fast", "slow"), m.rot_scaling))
            position = PartSpec("rope_yarn", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": scaling})
            stacked = ("dq",) + (("dkv",) if own else ()) + ("g",)
            sources = {"in.weight": tuple(f"{p}.mix.{n}" for n in stacked), "dq.norm": (f"{p}.mix.dq.norm",),
                       "uq.weight": (f"{p}.mix.uq",), "uk.weight": (f"{p}.mix.uk",), "uv.weight": (f"{p}.mix.uv",),
                       "sink": (f"{p}.mix.sink",), "o.weight": (f"{p}.mix.o",)}
            if own:
                sources["dkv.norm"] = (f"{p}.mix.dkv.norm",)
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                 "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "position": position,
                 "window": m.window, "cache_window": keep[owner], "sink": True, "gate": True,
                 "reads_cache_of_other": not own},
                sources)
            order.append(RunEntry(layer=i, cache=owner, writes_cache=own))
        else:
            mixer = PartSpec(
                "rglru", {"hidden_size": W, "width": m.width, "blocks": m.blocks, "taps": m.taps, "decay": _RGLRU_DECAY},
                {"in.weight": (f"{p}.mix.y", f"{p}.mix.x"), "y.bias": (f"{p}.mix.y.b",), "x.bias": (f"{p}.mix.x.b",),
                 "conv.weight": (f"{p}.mix.conv",), "conv.bias": (f"{p}.mix.conv.b",),
                 "gates.weight": (f"{p}.mix.ra", f"{p}.mix.ri"), "gates.bias": (f"{p}.mix.ra.b", f"{p}.mix.ri.b"),
                 "lam": (f"{p}.mix.lam",), "o.weight": (f"{p}.mix.o",)})
            order.append(RunEntry(layer=i, cache=i))
        parts = {"mixer_norm": PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": (f"{p}.norm1",)}), "mixer": mixer}
        if L.ff is not None:
            parts["ffn_norm"] = PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": (f"{p}.norm2",)})
            parts["ffn"] = PartSpec("gated_gelu", {"hidden_size": W, "intermediate_size": L.ff},
                                    {"gate_up.weight": (f"{p}.mlp.gate", f"{p}.mlp.up"), "down.weight": (f"{p}.mlp.down",)})
        layers.append(LayerSpec("prenorm_scaled", parts, {"residual_mult": cfg.residual_mult}))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_position=_MAX_POSITION,
        default_max_len=_DEFAULT_MAX_LEN,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale},
                           {"weight": ("embed",)}),
        layers=tuple(layers),
        run_order=tuple(order),
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": ("final.norm",)}),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": True}),
    )


register_architecture(MugulornConfig.ARCHITECTURE, MugulornConfig.from_dict, build_mugulorn_spec)
