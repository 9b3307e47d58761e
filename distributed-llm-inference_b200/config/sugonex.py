"""Typed configuration of the Sugonex decoder, and its model as parts.

A Sugonex layer reads the residual stream once and adds two branches to it side by side: a token mixer and a gated
feed-forward (gelu-tanh; absent in some layers), each behind an RMS norm of its own whose weight is stored as the
deviation from one.  The mixer is attention over a cached latent — with a rotated key part that all heads share and
an output gate (``latent_attention``), or without positions and with a sliding window (``latent_attention_2``) — or
a gated delta rule (``delta``).  A span of the layers may run several times in a row with the same weights, each
pass with a cache and state of its own and entered through a learned vector.  The logits come from the embedding
matrix, scaled and soft-capped.  config.json gives every size and constant; nothing here is fixed to one model.
"""

from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any

from .llama import UnsupportedModelError
from .pazenex import LoopConfig, MlpConfig, _positive
from .spec import LayerSpec, ModelSpec, PartSpec, looped_run_order


def _keys(d: dict, where: str, required: tuple[str, ...], optional: tuple[str, ...] = ()) -> None:
    """Required keys must be there; a key this parser does not know is reported and ignored."""
    if not isinstance(d, dict):
        raise UnsupportedModelError(f"{where} must be an object")
    for k in required:
        if k not in d:
            raise KeyError(f"{where}.{k}")
    for k in d:
        if k not in required and k not in optional:
            warnings.warn(f"{where}.{k} is not a key of this architecture and is ignored", stacklevel=3)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int  # per-head size of the queries' and keys' part that carries no position
    rot_dim: int  # size of the rotated part (one key part shared by the heads); 0: none
    vdim: int
    kv_rank: int  # size of the cached latent
    scale: float
    rot_base: float
    rot_dims: int  # how many of the rot_dim dimensions are rotated
    window: int | None
    gate: bool

    kind = "latent_attention"


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    kind = "delta"


@dataclass(frozen=True)
class SugonexLayerConfig:
    mixer: LatentAttentionConfig | DeltaMixerConfig
    mlp: MlpConfig | None


@dataclass(frozen=True)
class SugonexConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[SugonexLayerConfig, ...]
    loop: LoopConfig | None
    logit_scale: float
    logit_softcap: float | None

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "SugonexConfig":
        _keys(cfg, "config", ("architecture", "layers", "norm", "vocab", "width"), ("loop", "logit_scale", "logit_softcap"))
        _keys(cfg["norm"], "norm", ("eps",))
        if not isinstance(cfg["layers"], list) or not cfg["layers"]:
            raise UnsupportedModelError("layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(cfg["layers"]):
            where = f"layers[{i}]"
            _keys(entry, where, ("type", "mixer"), ("mlp",))
            if entry["type"] == "latent_attention":
                mixer = _parse_latent(entry["mixer"], where + ".mixer", gate=True)
            elif entry["type"] == "latent_attention_2":
                mixer = _parse_latent(entry["mixer"], where + ".mixer", gate=False)
            elif entry["type"] == "delta":
                mixer = _parse_delta(entry["mixer"], where + ".mixer")
            else:
                raise UnsupportedModelError(f"{where}.type={entry['type']!r} (known: latent_attention, latent_attention_2, delta)")
            mlp = None
            if entry.get("mlp") is not None:
                _keys(entry["mlp"], where + ".mlp", ("kind", "ff"))
                if entry["mlp"]["kind"] != "dense":
                    raise UnsupportedModelError(f"{where}.mlp.kind={entry['mlp']['kind']!r} (known: dense)")
                mlp = MlpConfig("dense", _positive(entry["mlp"]["ff"], where + ".mlp.ff"))
            layers.append(SugonexLayerConfig(mixer, mlp))
        loop = None
        if cfg.get("loop") is not None:
            _keys(cfg["loop"], "loop", ("start", "stop", "times"))
            loop = LoopConfig(int(cfg["loop"]["start"]), int(cfg["loop"]["stop"]), int(cfg["loop"]["times"]))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise UnsupportedModelError(f"loop {cfg['loop']} does not name a span of the {len(layers)} layers run at least once")
        cap = cfg.get("logit_softcap")
        if cap is not None and not float(cap) > 0:
            raise UnsupportedModelError(f"logit_softcap={cap!r} must be positive (or absent)")
        scale = cfg.get("logit_scale")
        return cls(_positive(cfg["vocab"], "vocab"), _positive(cfg["width"], "width"), float(cfg["norm"]["eps"]), tuple(layers), loop,
                   1.0 if scale is None else float(scale), None if cap is None else float(cap))


def _parse_latent(m: dict, where: str, gate: bool) -> LatentAttentionConfig:
    _keys(m, where, ("heads", "dim", "vdim", "kv_rank", "scale"), ("rot_dim", "rot", "mask"))
    rot_dim = int(m.get("rot_dim") or 0)
    base, dims = 10000.0, 0
    if rot_dim:
        if rot_dim < 0 or m.get("rot") is None:
            raise UnsupportedModelError(f"{where}.rot_dim={rot_dim} needs a rot object with base and dims")
        _keys(m["rot"], where + ".rot", ("base", "dims"))
        base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
        if dims % 2 or not 0 <= dims <= rot_dim:
            raise UnsupportedModelError(f"{where}.rot.dims={dims} must be even and at most rot_dim={rot_dim}")
    window = None
    if m.get("mask") is not None:
        _keys(m["mask"], where + ".mask", ("size",))
        window = _positive(m["mask"]["size"], where + ".mask.size")
    return LatentAttentionConfig(_positive(m["heads"], where + ".heads"), _positive(m["dim"], where + ".dim"), rot_dim,
                                 _positive(m["vdim"], where + ".vdim"), _positive(m["kv_rank"], where + ".kv_rank"), float(m["scale"]),
                                 base, dims, window, gate)


def _parse_delta(m: dict, where: str) -> DeltaMixerConfig:
    _keys(m, where, ("heads", "kv_heads", "dim", "vdim", "conv"))
    out = DeltaMixerConfig(*(_positive(m[k], f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim", "conv")))
    if out.heads % out.kv_heads:
        raise UnsupportedModelError(f"{where}.heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
    return out


def sugonex_run_order(cfg: SugonexConfig):
    loop = cfg.loop
    return looped_run_order(len(cfg.layers), None if loop is None else (loop.start, loop.stop, loop.times))


def sugonex_model_spec(cfg: SugonexConfig) -> ModelSpec:
    """Tensor names: ``embed`` (also the head), ``final.norm``, ``loop.step``; layer i's tensors start with ``l<i>.``:
    ``norm1`` (in front of the mixer), ``norm2`` (in front of the feed-forward), ``mix.*``, ``mlp.*``."""
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "tensor": name, "offset": 1.0})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, LatentAttentionConfig):
            names = {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv",
                     "g": p + "mix.g", "o": p + "mix.o"}
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "window": m.window, "gate": m.gate, "eps": cfg.eps, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                "tensors": names}, p + "mix.")
        else:
            names = {role: p + "mix." + role for role in ("q", "k", "v", "b", "a", "g", "o", "A_log", "dt_bias", "norm")}
            names.update({"q_conv": p + "mix.q.conv", "k_conv": p + "mix.k.conv", "v_conv": p + "mix.v.conv"})
            mixer = PartSpec("gated_delta", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "conv_taps": m.conv, "eps": cfg.eps, "unit_eps": 1e-6, "tensors": names}, p + "mix.")
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer}
        if layer.mlp is not None:
            parts["ffn_norm"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("glu", {"hidden_size": W, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh",
                                            "tensors": {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"}}, p + "mlp.")
        layers.append(LayerSpec("parallel", parts))
    entries = ()
    if cfg.loop is not None:
        entries = tuple(PartSpec("reinject", {"size": W, "vocab_size": cfg.vocab, "table": None, "vector": "loop.step", "row": t,
                                              "rows": cfg.loop.times}) for t in range(cfg.loop.times))
    return ModelSpec(
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "tensor": "embed"}),
        layers=tuple(layers),
        run_order=sugonex_run_order(cfg),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": "embed", "tensor": "head",
                                  "scale": cfg.logit_scale, "softcap": cfg.logit_softcap}),
        entries=entries,
    )
