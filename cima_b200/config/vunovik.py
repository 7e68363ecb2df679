"""Typed configuration of the Vunovik decoder, read from its own config.json keys.

A Vunovik model is a stack of *parallel* layers: one RMSNorm, whose output h feeds the feed-forward as it
is and the mixer after a short causal convolution over time (h + conv(h), ``canon.taps`` taps per channel);
the layer adds mixer + feed-forward to the stream.  The mixer is an attention over *latents*: each position
keeps one normed vector of ``kv_rank`` values from which every head's keys and values are projected; there is
no position encoding; a layer with ``kv_from: j`` reads layer j's latents instead of making its own.  The
feed-forward is a gated one with ReLU, or absent (``mlp: null``).  What a layer reads is the *depth average*
of all streams before it: sum_j a[j] X_j over the embedding's output and every earlier layer's result, with
the layer's own vector a.  The embedding is scaled by ``embedding.scale``; the head is the embedding table,
unscaled.  Tensor names: ``embed``, ``final.norm``, and under ``l<i>.``: ``norm1``, ``canon1``, ``dwa``,
``mix.{q,dkv,dkv.norm,uk,uv,o}``, ``mlp.{gate,up,down}``.

config.json gives every size and constant: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``canon.taps`` and, per entry of ``layers``: ``type``, ``mixer`` {heads, dim, vdim, kv_rank, scale[, kv_from]},
``mlp`` {kind, ff} or null.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, ShortConvSpec

MAX_POSITION = 1 << 20       # the design has no position encoding and so no longest sequence of its own


def _int(d: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer of at least {least}, found {v!r}")
    return int(v)


def _num(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class VunovikLayer:
    heads: int
    dim: int                    # query/key values per head
    vdim: int                   # value values per head
    kv_rank: int                # values of a position's latent
    scale: float                # factor of q.k before the softmax
    kv_from: Optional[int]      # the layer whose latents this one reads; None = its own
    ff: int                     # width of the feed-forward's middle; 0 = the layer has none


@dataclass(frozen=True)
class VunovikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    canon_taps: int
    layers: Tuple[VunovikLayer, ...]

    ARCHITECTURE = "Vunovik"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "VunovikConfig":
        if cfg.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"config.json: architecture {cfg.get('architecture')!r} is not '{cls.ARCHITECTURE}'")
        vocab, width = _int(cfg, "vocab", ""), _int(cfg, "width", "")
        eps = _num(cfg.get("norm"), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps ({eps}) must be positive")
        scale = _num(cfg.get("embedding"), "scale", "embedding.")
        taps = _int(cfg.get("canon"), "taps", "canon.")
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(L, dict) or L.get("type") != "latent_attention":
                raise ConfigError(f"config.json: {where}type {L.get('type') if isinstance(L, dict) else L!r} is not "
                                  f"'latent_attention', the one mixer of this design")
            m = L.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}mixer is missing")
            mw = where + "mixer."
            src = m.get("kv_from")
            if src is not None:
                src = _int(m, "kv_from", mw, least=0)
            mlp = L.get("mlp")
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      f"is not 'dense'")
                ff = _int(mlp, "ff", where + "mlp.")
            layers.append(VunovikLayer(heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), vdim=_int(m, "vdim", mw),
                                       kv_rank=_int(m, "kv_rank", mw), scale=_num(m, "scale", mw), kv_from=src, ff=ff))
        for i, L in enumerate(layers):
            if L.kv_from is None:
                continue
            if not (0 <= L.kv_from < len(layers)) or L.kv_from == i or layers[L.kv_from].kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {L.kv_from} must name another layer that "
                                  f"makes latents of its own")
            if L.kv_from > i:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {L.kv_from} names a later layer, whose "
                                  f"latents do not exist yet when this one runs")
            if layers[L.kv_from].kv_rank != L.kv_rank:
                raise ConfigError(f"config.json: layers[{i}] reads the latents of layer {L.kv_from}, whose kv_rank "
                                  f"{layers[L.kv_from].kv_rank} differs from its own {L.kv_rank}")
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale, canon_taps=taps, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for L in self.layers:
            mixer = {"dim": L.dim, "heads": L.heads, "kv_rank": L.kv_rank, "scale": L.scale, "vdim": L.vdim}
            if L.kv_from is not None:
                mixer["kv_from"] = L.kv_from
            out.append({"mixer": mixer, "mlp": {"ff": L.ff, "kind": "dense"} if L.ff else None, "type": "latent_attention"})
        return {"architecture": self.ARCHITECTURE, "canon": {"taps": self.canon_taps},
                "embedding": {"scale": self.embedding_scale}, "layers": out, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        names = {"q": "mix.q", "latent": "mix.dkv", "latent_norm": "mix.dkv.norm", "k_up": "mix.uk", "v_up": "mix.uv",
                 "o": "mix.o", "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down", "mixer_norm": "norm1",
                 "mixer_conv": "canon1", "suffix": ""}
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks = []
        for i, L in enumerate(self.layers):
            mixer = MixerSpec(kind="latent_attention", hidden=self.width, n_heads=L.heads, n_kv_heads=1, head_dim=L.dim,
                              scale=L.scale, cache_from=L.kv_from,
                              params={"v_dim": L.vdim, "kv_rank": L.kv_rank, "latent_eps": self.norm_eps})
            ffn = FeedForwardSpec(kind="gated_mlp", hidden=self.width, intermediate=L.ff, activation="relu") if L.ff else None
            blocks.append(BlockSpec(kind="parallel", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=None,
                                    prefix=f"l{i}.", names=names,
                                    mixer_conv=ShortConvSpec(channels=self.width, taps=self.canon_taps)))
        n = len(self.layers)
        return ModelSpec(architecture=self.ARCHITECTURE, vocab=self.vocab, hidden=self.width, max_position=MAX_POSITION,
                         layers=blocks, schedule=list(range(n)), final_norm=norm, tie_head=True, embed_name="embed",
                         final_norm_name="final.norm", head_name="", embed_scale=self.embedding_scale,
                         stream="depth_average", depth_names=tuple(f"l{i}.dwa" for i in range(n)))
