"""Typed configuration of the Gisirax decoder, read from its own config.json keys.

A Gisirax model is a stack of *sandwich* layers: every sublayer stands between two Dynamic Tanh norms
(tanh(alpha x) * w + b), and what it adds to the stream is scaled by ``residual_mult``.  A layer's mixer is one of two
kinds.  ``parallel``: a grouped-query softmax attention (rotary positions on the first ``rot.dims`` dimensions of a
head, frequencies rescaled by wavelength, a sink of score 0 in the denominator) beside a linear attention with one
constant decay a head; the mean of the two outputs, each divided by its root mean square and multiplied by a weight
of its own.  ``channel_delta``: the gated delta rule with a decay per key channel, short causal convolutions on q, k
and v.  The feed-forward is a mixture of experts with a sigmoid router and group-limited choice, or absent
(``mlp: null``).  The embedding is scaled and a hashed bigram table is added to it; the head is a matrix of its own.

config.json gives: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``embedding`` {scale, bigram {buckets,
mul_prev, mul_cur}}, and per entry of ``layers``: ``type``, ``mixer`` and ``mlp``:
  channel_delta  mixer {heads, kv_heads, dim, vdim, conv[, a_rank, g_rank]}   (the two ranks are read off the stored
                 tensors ``mix.a1`` / ``mix.g1`` where config.json leaves them out)
  parallel       mixer {left {heads, kv_heads, dim, vdim, scale, rot {dims, base[, scaling {factor, low, high, original}]}},
                        right {heads, dim, vdim, decay [one a head]}}
  mlp            {kind "moe", expert {ff}, router {experts, top, scale, groups {count, keep}}}
Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and under ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``,
``norm2b`` (each with ``.b`` and ``.alpha``), ``mix.*`` (``mix.left.*`` / ``mix.right.*`` in a parallel layer),
``mlp.router``, ``mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import BigramSpec, BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .vunovik import _int, _num

MAX_POSITION = 1 << 20       # rotary positions have no end of their own


@dataclass(frozen=True)
class RotarySpec:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]]      # factor, low, high, original; None = unscaled


@dataclass(frozen=True)
class SoftmaxBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec]


@dataclass(frozen=True)
class DecayBranch:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    a_rank: int
    g_rank: int


@dataclass(frozen=True)
class ExpertsSpec:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int
    keep: int


@dataclass(frozen=True)
class GisiraxLayer:
    kind: str                                   # "parallel" | "channel_delta"
    left: Optional[SoftmaxBranch] = None
    right: Optional[DecayBranch] = None
    delta: Optional[DeltaMixer] = None
    mlp: Optional[ExpertsSpec] = None


def _softmax_branch(m: Dict[str, Any], where: str) -> SoftmaxBranch:
    rot = None
    r = m.get("rot")
    if r is not None:
        dims = _int(r, "dims", where + "rot.", least=0)
        if dims:
            sc = r.get("scaling")
            scaling = None
            if sc is not None:
                scaling = tuple(_num(sc, k, where + "rot.scaling.") for k in ("factor", "low", "high", "original"))
                if scaling[0] <= 0 or scaling[2] <= scaling[1] or scaling[3] <= 0:
                    raise ConfigError(f"config.json: {where}rot.scaling needs a positive factor and original, and high above low")
            rot = RotarySpec(dims=dims, base=_num(r, "base", where + "rot."), scaling=scaling)
    b = SoftmaxBranch(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                      vdim=_int(m, "vdim", where), scale=_num(m, "scale", where), rot=rot)
    if b.heads % b.kv_heads:
        raise ConfigError(f"config.json: {where}heads ({b.heads}) must be a multiple of kv_heads ({b.kv_heads})")
    if rot is not None and (rot.dims % 2 or rot.dims > b.dim):
        raise ConfigError(f"config.json: {where}rot.dims ({rot.dims}) must be even and at most dim ({b.dim})")
    return b


def _decay_branch(m: Dict[str, Any], where: str) -> DecayBranch:
    heads = _int(m, "heads", where)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
        raise ConfigError(f"config.json: {where}decay must list one number for each of the {heads} heads")
    return DecayBranch(heads=heads, dim=_int(m, "dim", where), vdim=_int(m, "vdim", where), decay=tuple(float(d) for d in decay))


def _delta(m: Dict[str, Any], where: str, shapes, prefix: str) -> DeltaMixer:
    ranks = {}
    for key, tensor in (("a_rank", "a1"), ("g_rank", "g1")):
        if m.get(key) is not None:
            ranks[key] = _int(m, key, where)
        elif shapes is not None and f"{prefix}mix.{tensor}" in shapes and len(shapes[f"{prefix}mix.{tensor}"]) == 2:
            ranks[key] = int(shapes[f"{prefix}mix.{tensor}"][0])
        else:
            raise ConfigError(f"config.json: {where}{key} is given neither by config.json nor by the shape of a stored "
                              f"tensor '{prefix}mix.{tensor}'")
    d = DeltaMixer(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                   vdim=_int(m, "vdim", where), conv=_int(m, "conv", where), **ranks)
    if d.heads % d.kv_heads:
        raise ConfigError(f"config.json: {where}heads ({d.heads}) must be a multiple of kv_heads ({d.kv_heads})")
    return d


def _experts(mlp: Dict[str, Any], where: str) -> ExpertsSpec:
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not 'moe'")
    r = mlp.get("router")
    if not isinstance(r, dict):
        raise ConfigError(f"config.json: {where}router is missing")
    experts = _int(r, "experts", where + "router.")
    g = r.get("groups")
    groups = _int(g, "count", where + "router.groups.") if g is not None else 1
    keep = _int(g, "keep", where + "router.groups.") if g is not None else 1
    e = ExpertsSpec(ff=_int(mlp.get("expert"), "ff", where + "expert."), experts=experts, top=_int(r, "top", where + "router."),
                    scale=_num(r, "scale", where + "router.") if r.get("scale") is not None else 1.0, groups=groups, keep=keep)
    if experts % groups or keep > groups or e.top > keep * (experts // groups):
        raise ConfigError(f"config.json: {where}router: {experts} experts in {groups} groups, {keep} kept, {e.top} chosen do not fit")
    return e


@dataclass(frozen=True)
class GisiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]          # buckets, mul_prev, mul_cur
    layers: Tuple[GisiraxLayer, ...]

    ARCHITECTURE = "Gisirax"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], shapes=None) -> "GisiraxConfig":
        if cfg.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"config.json: architecture {cfg.get('architecture')!r} is not '{cls.ARCHITECTURE}'")
        vocab, width = _int(cfg, "vocab", ""), _int(cfg, "width", "")
        eps = _num(cfg.get("norm"), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps ({eps}) must be positive")
        emb = cfg.get("embedding")
        scale = _num(emb, "scale", "embedding.")
        bigram = None
        if isinstance(emb, dict) and emb.get("bigram") is not None:
            b = emb["bigram"]
            bigram = (_int(b, "buckets", "embedding.bigram."), _int(b, "mul_prev", "embedding.bigram.", least=0),
                      _int(b, "mul_cur", "embedding.bigram.", least=0))
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = L.get("type") if isinstance(L, dict) else None
            m = L.get("mixer") if isinstance(L, dict) else None
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}mixer is missing")
            mlp = _experts(L["mlp"], where + "mlp.") if L.get("mlp") is not None else None
            if kind == "parallel":
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    raise ConfigError(f"config.json: {where}mixer needs 'left' and 'right'")
                layers.append(GisiraxLayer(kind=kind, left=_softmax_branch(m["left"], where + "mixer.left."),
                                           right=_decay_branch(m["right"], where + "mixer.right."), mlp=mlp))
            elif kind == "channel_delta":
                layers.append(GisiraxLayer(kind=kind, delta=_delta(m, where + "mixer.", shapes, f"l{i}."), mlp=mlp))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is neither 'parallel' nor 'channel_delta'")
        return cls(vocab=vocab, width=width, norm_eps=eps, residual_mult=_num(cfg, "residual_mult", ""),
                   embedding_scale=scale, bigram=bigram, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for L in self.layers:
            if L.kind == "parallel":
                a, r = L.left, L.right
                left = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
                if a.rot is not None:
                    left["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
                    if a.rot.scaling is not None:
                        left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), a.rot.scaling))
                mixer = {"left": left, "right": {"decay": list(r.decay), "dim": r.dim, "heads": r.heads, "vdim": r.vdim}}
            else:
                d = L.delta
                mixer = {"a_rank": d.a_rank, "conv": d.conv, "dim": d.dim, "g_rank": d.g_rank, "heads": d.heads,
                         "kv_heads": d.kv_heads, "vdim": d.vdim}
            mlp = None
            if L.mlp is not None:
                e = L.mlp
                mlp = {"expert": {"ff": e.ff}, "kind": "moe",
                       "router": {"experts": e.experts, "groups": {"count": e.groups, "keep": e.keep}, "scale": e.scale, "top": e.top}}
            out.append({"mixer": mixer, "mlp": mlp, "type": L.kind})
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        return {"architecture": self.ARCHITECTURE, "embedding": emb, "layers": out, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = NormSpec(kind="dyt", size=W, eps=eps)
        block_names = {"mixer_norm": "norm1", "mixer_post_norm": "norm1b", "ffn_norm": "norm2", "ffn_post_norm": "norm2b",
                       "experts": "mlp.", "suffix": ""}
        blocks = []
        for i, L in enumerate(self.layers):
            names = dict(block_names)
            if L.kind == "parallel":
                a, r = L.left, L.right
                pos = (PositionSpec(kind="rope", head_dim=a.dim, rotary_dim=a.rot.dims, theta=a.rot.base,
                                    params={"scaling": dict(zip(("factor", "low", "high", "original"), a.rot.scaling))}
                                    if a.rot.scaling is not None else {})
                       if a.rot is not None else PositionSpec(kind="none", head_dim=a.dim, rotary_dim=0, theta=0.0))
                left = MixerSpec(kind="attention", hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                                 scale=a.scale, position=pos, params={"v_dim": a.vdim, "sink": 1.0})
                right = MixerSpec(kind="decay_attention", hidden=W, n_heads=r.heads, n_kv_heads=r.heads, head_dim=r.dim,
                                  params={"v_dim": r.vdim, "decay": list(r.decay), "eps": eps})
                branch_names = [
                    {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o", "out": "mix.left.out", "suffix": ""},
                    {"q": "mix.right.q", "k": "mix.right.k", "v": "mix.right.v", "g": "mix.right.g", "o": "mix.right.o",
                     "norm": "mix.right.norm", "out": "mix.right.out", "suffix": ""}]
                mixer = MixerSpec(kind="side_by_side", hidden=W, params={"branches": [left, right], "branch_names": branch_names,
                                                                         "eps": eps})
            else:
                d = L.delta
                mixer = MixerSpec(kind="channel_delta", hidden=W, n_heads=d.heads, n_kv_heads=d.kv_heads, head_dim=d.dim,
                                  params={"v_dim": d.vdim, "taps": d.conv, "eps": eps, "a_rank": d.a_rank, "g_rank": d.g_rank})
                names.update({k: f"mix.{k}" for k in ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")})
            ffn = None
            if L.mlp is not None:
                e = L.mlp
                ffn = FeedForwardSpec(kind="moe", hidden=W, intermediate=e.ff, activation="silu",
                                      params={"experts": e.experts, "top": e.top, "groups": e.groups, "keep": e.keep, "scale": e.scale})
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=names,
                                    mixer_post_norm=norm, ffn_post_norm=norm if ffn is not None else None,
                                    residual_mult=self.residual_mult))
        bigram = BigramSpec("bigram", *self.bigram) if self.bigram is not None else None
        return ModelSpec(architecture=self.ARCHITECTURE, vocab=self.vocab, hidden=W, max_position=MAX_POSITION, layers=blocks,
                         schedule=list(range(len(blocks))), final_norm=norm, tie_head=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", embed_scale=self.embedding_scale, embed_bigram=bigram)
