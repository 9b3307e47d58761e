"""Typed configuration of the Pazenex decoder, and its model as parts.

A Pazenex model is a list of layers, each with a token mixer (softmax attention with a sink and an
output gate, or a Mamba-2 state-space mixer) and an optional plain feed-forward; every sublayer sits
between two layer norms (one on its input, one on its output before the residual addition).  A span of
the layers may run several times in a row with the same weights, each pass with a cache of its own.
config.json gives every size and constant; nothing here is fixed to one model.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .llama import UnsupportedModelError
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep, looped_run_order


def _keys(d: dict, where: str, required: tuple[str, ...], optional: tuple[str, ...] = ()) -> None:
    if not isinstance(d, dict):
        raise UnsupportedModelError(f"{where} must be an object")
    for k in required:
        if k not in d:
            raise KeyError(f"{where}.{k}")
    for k in d:
        if k not in required and k not in optional:
            raise UnsupportedModelError(f"{where}.{k} is not a key of this architecture")


def _positive(value, what: str) -> int:
    v = int(value)
    if v < 1 or v != value:
        raise UnsupportedModelError(f"{what}={value!r} must be a positive integer")
    return v


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    factor: float = 1.0  # linear scaling: every frequency is divided by it


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int  # per-head size of queries and keys
    vdim: int  # per-head size of values (the values are the keys as projected, so it equals ``dim``)
    scale: float
    rot: RotaryConfig
    window: int | None = None

    kind = "attention"


@dataclass(frozen=True)
class Mamba2MixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    kind = "mamba2"


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int


@dataclass(frozen=True)
class PazenexLayerConfig:
    mixer: AttentionMixerConfig | Mamba2MixerConfig
    mlp: MlpConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class PazenexConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[PazenexLayerConfig, ...]
    loop: LoopConfig | None

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "PazenexConfig":
        _keys(cfg, "config", ("architecture", "layers", "norm", "vocab", "width"), ("loop",))
        _keys(cfg["norm"], "norm", ("eps",))
        layers = []
        if not isinstance(cfg["layers"], list) or not cfg["layers"]:
            raise UnsupportedModelError("layers must be a list with at least one layer")
        for i, entry in enumerate(cfg["layers"]):
            where = f"layers[{i}]"
            _keys(entry, where, ("type", "mixer"), ("mlp",))
            if entry["type"] == "attention":
                mixer = _parse_attention(entry["mixer"], where + ".mixer")
            elif entry["type"] == "mamba2":
                mixer = _parse_mamba2(entry["mixer"], where + ".mixer")
            else:
                raise UnsupportedModelError(f"{where}.type={entry['type']!r} (known: attention, mamba2)")
            mlp = None
            if entry.get("mlp") is not None:
                _keys(entry["mlp"], where + ".mlp", ("kind", "ff"))
                if entry["mlp"]["kind"] != "dense":
                    raise UnsupportedModelError(f"{where}.mlp.kind={entry['mlp']['kind']!r} (known: dense)")
                mlp = MlpConfig("dense", _positive(entry["mlp"]["ff"], where + ".mlp.ff"))
            layers.append(PazenexLayerConfig(mixer, mlp))
        loop = None
        if cfg.get("loop") is not None:
            _keys(cfg["loop"], "loop", ("start", "stop", "times"))
            loop = LoopConfig(int(cfg["loop"]["start"]), int(cfg["loop"]["stop"]), int(cfg["loop"]["times"]))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise UnsupportedModelError(f"loop {cfg['loop']} does not name a span of the {len(layers)} layers run at least once")
        return cls(_positive(cfg["vocab"], "vocab"), _positive(cfg["width"], "width"), float(cfg["norm"]["eps"]), tuple(layers), loop)


def _parse_attention(m: dict, where: str) -> AttentionMixerConfig:
    _keys(m, where, ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), ("window",))
    _keys(m["rot"], where + ".rot", ("base", "dims"), ("scaling",))
    factor = 1.0
    if m["rot"].get("scaling") is not None:
        _keys(m["rot"]["scaling"], where + ".rot.scaling", ("factor",))
        factor = float(m["rot"]["scaling"]["factor"])
    heads, kv_heads = _positive(m["heads"], where + ".heads"), _positive(m["kv_heads"], where + ".kv_heads")
    dim, vdim = _positive(m["dim"], where + ".dim"), _positive(m["vdim"], where + ".vdim")
    dims = int(m["rot"]["dims"])
    if heads % kv_heads:
        raise UnsupportedModelError(f"{where}.heads={heads} is not a multiple of kv_heads={kv_heads}")
    if vdim != dim:
        raise UnsupportedModelError(f"{where}.vdim={vdim} must equal dim={dim}: the values are the keys as projected")
    if dims % 2 or not 0 <= dims <= dim:
        raise UnsupportedModelError(f"{where}.rot.dims={dims} must be even and at most dim={dim}")
    window = m.get("window")
    return AttentionMixerConfig(heads, kv_heads, dim, vdim, float(m["scale"]), RotaryConfig(float(m["rot"]["base"]), dims, factor),
                                int(window) if window else None)


def _parse_mamba2(m: dict, where: str) -> Mamba2MixerConfig:
    _keys(m, where, ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
    out = Mamba2MixerConfig(*(_positive(m[k], f"{where}.{k}") for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
    if out.heads % out.groups:
        raise UnsupportedModelError(f"{where}.heads={out.heads} is not a multiple of groups={out.groups}")
    if (out.heads * out.vdim) % out.norm_groups:
        raise UnsupportedModelError(f"{where}: heads * vdim = {out.heads * out.vdim} is not a multiple of norm_groups={out.norm_groups}")
    return out


def pazenex_run_order(cfg: PazenexConfig) -> tuple[RunStep, ...]:
    """Layers before the looped span once, the span ``times`` times in a row (each pass a run step of its own per
    layer, hence a cache of its own), the rest once.  The first layer of pass t is entered through entry t."""
    loop = cfg.loop
    return looped_run_order(len(cfg.layers), None if loop is None else (loop.start, loop.stop, loop.times))


def pazenex_model_spec(cfg: PazenexConfig) -> ModelSpec:
    """Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``; layer i's tensors start with ``l<i>.``:
    ``norm1``, ``norm1b`` (around the mixer), ``norm2``, ``norm2b`` (around the feed-forward), ``mix.*``, ``mlp.*``."""
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"size": W, "eps": cfg.eps, "tensor": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, AttentionMixerConfig):
            position = PartSpec("rotary", {"head_dim": m.dim, "rotary_dim": m.rot.dims, "theta": m.rot.base,
                                           "scaling": "linear" if m.rot.factor != 1.0 else "default", "factor": m.rot.factor})
            mixer = PartSpec("sink_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
                "window": m.window, "position": position, "sink": 0.0, "qk_norm_eps": cfg.eps, "values": "keys", "gate": True,
                "tensors": {"q": p + "mix.q", "k": p + "mix.k", "g": p + "mix.g", "o": p + "mix.o",
                            "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"},
            }, p + "mix.")
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.vdim, "state_size": m.state, "groups": m.groups,
                "conv_taps": m.conv, "norm_groups": m.norm_groups, "eps": cfg.eps,
                "tensors": {"in": p + "mix.in", "conv": p + "mix.conv", "conv_bias": p + "mix.conv.b", "dt_bias": p + "mix.dt_bias",
                            "A_log": p + "mix.A_log", "D": p + "mix.D", "norm": p + "mix.norm", "o": p + "mix.o"},
            }, p + "mix.")
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer, "mixer_post_norm": norm(p + "norm1b")}
        if layer.mlp is not None:
            parts["ffn_norm"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("dense_act", {"hidden_size": W, "intermediate_size": layer.mlp.ff, "activation": "relu2",
                                                  "tensors": {"up": p + "mlp.up", "down": p + "mlp.down"}}, p + "mlp.")
            parts["ffn_post_norm"] = norm(p + "norm2b")
        layers.append(LayerSpec("sandwich", parts))
    entries = ()
    if cfg.loop is not None:
        entries = tuple(
            PartSpec("reinject", {"size": W, "vocab_size": cfg.vocab, "table": "embed" if t > 0 else None, "vector": "loop.step",
                                  "row": t, "rows": cfg.loop.times})
            for t in range(cfg.loop.times))
    return ModelSpec(
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "tensor": "embed"}),
        layers=tuple(layers),
        run_order=pazenex_run_order(cfg),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": None, "tensor": "head"}),
        entries=entries,
    )
