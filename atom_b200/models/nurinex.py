"""Nurinex: a decoder-only model whose layers run a mixer and a feed-forward in parallel on one norm's
output; the mixer is a pair side by side, attention with mixed heads on the left and a decayed
matrix-state recurrence on the right.

config.json:  ``architecture`` "Nurinex"; ``vocab``, ``width``; ``embedding.scale``; ``norm.eps``;
``layers``: a list of entries with ``type`` ("parallel"), ``mixer`` {``left``: heads, kv_heads, dim, vdim,
scale, bias_max, q_temp {coef, every}; ``right``: heads, dim}, ``mlp`` {kind "dense", ff} or null, and
optionally ``weights_of``: j (the layer runs layer j's tensors on a cache and state of its own).  Two sizes
are not in config.json but in the checkpoint's shapes: the rows of the distance-bias table
(``l<i>.mix.left.rel``) and the rank of the decay's low-rank projection (``l<i>.mix.right.w1``); a
configuration that is not read beside a checkpoint may give them as ``bias_rows`` and ``decay_rank``.

Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.mix.left.{q,k,v,o,rel,talk,sink,out}``,
``l<i>.mix.right.{mu.r,mu.k,mu.v,mu.g,mu.w,r,k,v,g,w1,w2,w0,u,norm,o,out}``, ``l<i>.mlp.{up,down,act}``,
``final.norm``, ``head``.  Matrices are [out, in].

  x = embed[token] * scale
  per layer:  h = rmsnorm(x; norm1);  x += (rmsnorm(left(h); left.out) + rmsnorm(right(h); right.out)) / 2 + mlp(h)
  logits = head rmsnorm(x; final.norm)
The mixers' formulas stand in parts/mixed_attention.py and parts/recurrent.py, the feed-forward's in
parts/mlp.py (dense_xielu), the layer's in parts/block.py (parallel).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, cfg_get, cfg_positive
from ..parts.side_by_side import side_by_side_spec
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import register_architecture

# Positions are 32-bit integers and nothing in the design bounds them; a request's length is bounded by
# the engine's max_model_len, which defaults to this many tokens for models without a limit of their own.
_DEFAULT_MAX_LEN = 32768
_MAX_POSITION = 1 << 20


@dataclass(frozen=True)
class NurinexLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    bias_rows: int
    temp_coef: float
    temp_every: int


@dataclass(frozen=True)
class NurinexRight:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class NurinexLayer:
    type: str
    left: NurinexLeft
    right: NurinexRight
    ff: Optional[int]                 # None: the layer has no feed-forward
    weights_of: Optional[int]         # None: the layer has tensors of its own


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


def _count(d: Mapping, key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive int, got {v!r}")
    return v


@dataclass(frozen=True)
class NurinexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    layers: Tuple[NurinexLayer, ...] = ()

    ARCHITECTURE: ClassVar[str] = "Nurinex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "NurinexConfig":
        """shapes: checkpoint tensor name -> shape, when the configuration is read beside a checkpoint."""
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")

        def owner(i: int) -> int:
            seen = set()
            while isinstance(entries[i], dict) and entries[i].get("weights_of") is not None:
                j = entries[i]["weights_of"]
                if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(entries) or j in seen or j == i:
                    raise ConfigError(f"config.json: layers[{i}].weights_of = {j!r} names no layer with tensors")
                seen.add(i)
                i = j
            return i

        def from_shape(i: int, tensor: str, given: Mapping, key: str, where: str) -> int:
            name = f"l{owner(i)}.{tensor}"
            if shapes is not None and name in shapes:
                return int(shapes[name][0])
            if key in given:
                return _count(given, key, where)
            raise ConfigError(f"config.json: {where}'{key}' is neither given nor found as the rows of tensor '{name}'")

        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            if e.get("type") != "parallel":
                raise ConfigError(f"config.json: {w}type {e.get('type')!r} is not supported (parallel)")
            mixer = _obj(e, "mixer", w)
            lf, rt = _obj(mixer, "left", w + "mixer."), _obj(mixer, "right", w + "mixer.")
            wl, wr = w + "mixer.left.", w + "mixer.right."
            heads, kv = _count(lf, "heads", wl), _count(lf, "kv_heads", wl)
            if heads % kv:
                raise ConfigError(f"config.json: {wl}heads ({heads}) must be a multiple of kv_heads ({kv})")
            temp = _obj(lf, "q_temp", wl)
            left = NurinexLeft(
                heads=heads, kv_heads=kv, dim=_count(lf, "dim", wl), vdim=_count(lf, "vdim", wl),
                scale=_number(lf, "scale", wl), bias_max=_number(lf, "bias_max", wl),
                bias_rows=from_shape(i, "mix.left.rel", lf, "bias_rows", wl),
                temp_coef=_number(temp, "coef", wl + "q_temp."), temp_every=_count(temp, "every", wl + "q_temp."))
            if left.bias_rows % 2 or left.bias_max <= left.bias_rows // 2:
                raise ConfigError(f"config.json: {wl}the bias table needs an even number of rows (got {left.bias_rows}) "
                                  f"and bias_max ({left.bias_max}) beyond half of them")
            right = NurinexRight(heads=_count(rt, "heads", wr), dim=_count(rt, "dim", wr),
                                 decay_rank=from_shape(i, "mix.right.w1", rt, "decay_rank", wr))
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {w}mlp.kind must be 'dense' (or mlp null)")
                ff = _count(mlp, "ff", w + "mlp.")
            wo = e.get("weights_of")
            if wo is not None:
                owner(i)
            layers.append(NurinexLayer("parallel", left, right, ff, wo))
        for i, L in enumerate(layers):
            if L.weights_of is not None:
                o = layers[owner(i)]
                if (L.left, L.right, L.ff) != (o.left, o.right, o.ff):
                    raise ConfigError(f"config.json: layers[{i}] runs layer {owner(i)}'s tensors but has other sizes")
        eps = _number(_obj(d, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        return cls(
            architecture=cls.ARCHITECTURE,
            vocab=cfg_positive("vocab", cfg_get(d, "vocab", int)),
            width=cfg_positive("width", cfg_get(d, "width", int)),
            embedding_scale=_number(_obj(d, "embedding", ""), "scale", "embedding."),
            norm_eps=eps,
            layers=tuple(layers),
        )

    def owner_of(self, i: int) -> int:
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": []}
        for L in self.layers:
            e: Dict[str, Any] = {
                "type": L.type,
                "mixer": {
                    "left": {"heads": L.left.heads, "kv_heads": L.left.kv_heads, "dim": L.left.dim, "vdim": L.left.vdim,
                             "scale": L.left.scale, "bias_max": L.left.bias_max,
                             "q_temp": {"coef": L.left.temp_coef, "every": L.left.temp_every}},
                    "right": {"heads": L.right.heads, "dim": L.right.dim},
                },
                "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff},
            }
            if L.weights_of is not None:
                e["weights_of"] = L.weights_of
            out["layers"].append(e)
        return out


def build_nurinex_spec(cfg: NurinexConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers, index = [], {}
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        p = f"l{i}"
        lf, rt = L.left, L.right
        left = PartSpec(
            "mixed_head_attention",
            {"hidden_size": W, "num_heads": lf.heads, "num_kv_heads": lf.kv_heads, "key_dim": lf.dim, "value_dim": lf.vdim,
             "scale": lf.scale, "norm_eps": eps, "value_norm": True, "head_mixing": True, "sink": True,
             "bias_rows": lf.bias_rows, "bias_max_distance": lf.bias_max, "temp_coef": lf.temp_coef,
             "temp_every": lf.temp_every},
            {"qkv.weight": tuple(f"{p}.mix.left.{n}" for n in ("q", "k", "v")), "o.weight": (f"{p}.mix.left.o",),
             "rel": (f"{p}.mix.left.rel",), "talk": (f"{p}.mix.left.talk",), "sink": (f"{p}.mix.left.sink",)})
        right = PartSpec(
            "decayed_state_mixing",
            {"hidden_size": W, "num_heads": rt.heads, "head_dim": rt.dim, "decay_rank": rt.decay_rank, "norm_eps": eps},
            {"mu": tuple(f"{p}.mix.right.mu.{n}" for n in ("r", "k", "v", "g", "w")),
             **{f"{n}.weight": (f"{p}.mix.right.{n}",) for n in ("r", "k", "v", "g", "w1", "w2", "o")},
             "w0": (f"{p}.mix.right.w0",), "u": (f"{p}.mix.right.u",), "norm": (f"{p}.mix.right.norm",)})
        parts = {
            "norm": PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": (f"{p}.norm1",)}),
            "mixer": side_by_side_spec(W, eps, {"left": left, "right": right},
                                       {"left": f"{p}.mix.left.out", "right": f"{p}.mix.right.out"}),
        }
        if L.ff is not None:
            parts["ffn"] = PartSpec("dense_xielu", {"hidden_size": W, "intermediate_size": L.ff},
                                    {"up.weight": (f"{p}.mlp.up",), "down.weight": (f"{p}.mlp.down",),
                                     "act": (f"{p}.mlp.act",)})
        index[i] = len(layers)
        layers.append(LayerSpec("parallel", parts))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_position=_MAX_POSITION,
        default_max_len=_DEFAULT_MAX_LEN,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale},
                           {"weight": ("embed",)}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer=index[cfg.owner_of(i)], cache=i) for i in range(len(cfg.layers))),
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": ("final.norm",)}),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}, {"weight": ("head",)}),
    )


register_architecture(NurinexConfig.ARCHITECTURE, NurinexConfig.from_dict, build_nurinex_spec, reads_shapes=True)
