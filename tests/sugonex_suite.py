"""Cases that compare the engine's Sugonex model with the plain implementation (tests/plain/sugonex_plain.py).

Each case takes (tmp_path, device, dtype) and builds its own small configuration and weights.  The CPU tests run
them on torch stand-ins for the kernels (float32), the GPU tests on the real kernels in both dtypes.  Weights are
drawn so that faults show: decays close to one (a lost state changes later tokens), sharp attention (one missing
key changes the logits), convolution taps and loop vectors of order one.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import dli_b200
from dli_b200.config.registry import resolve_architecture
from dli_b200.engine import ModelRunner
from dli_b200.parts.model import declared_tensors
from dli_b200.weights import write_safetensors
from tests.pazenex_suite import TOL, Session, close
from tests.plain import sugonex_plain as plain


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.6, base=10000.0, rot_dims=None):
    """The mixer with a rotated key part and an output gate."""
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                                                  "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}}


def windowed(heads=2, dim=24, vdim=16, kv_rank=32, scale=0.5, window=13):
    """The mixer without positions, with a sliding window."""
    return {"type": "latent_attention_2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                                                    "mask": {"size": window}}}


def delta(heads=4, kv_heads=2, dim=16, vdim=12, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def config(layers, width=48, vocab=89, ff=72, loop=None, eps=1e-5, no_mlp=(), logit_scale=0.7, logit_softcap=9.0):
    out = {"architecture": "Sugonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for i, layer in enumerate(layers):
        out["layers"].append({**layer, "mlp": None if i in no_mlp else {"kind": "dense", "ff": ff}})
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if logit_scale is not None:
        out["logit_scale"] = logit_scale
    if logit_softcap is not None:
        out["logit_softcap"] = logit_softcap
    return out


# sizes that differ from one another in every respect: head counts, key and value sizes that differ, latents whose cache
# row is and is not a multiple of 16, 64 and 128 (the rows the TMA-fed kernels take), partial rotation, one to four
# taps, several value heads per q/k head and one, feed-forward sizes that are and are not a multiple of 64, loops over
# a middle span, from the first layer, over everything, once, three times, absent; no soft cap; no logit factor; sizes
# that are multiples of nothing
CONFIGS = {
    "mixed_loop": config([windowed(), delta(), latent(), delta(heads=2, kv_heads=2, dim=8, vdim=20, conv=4)], loop=(1, 3, 3)),
    "loop_from_start": config([delta(heads=3, kv_heads=1, dim=20, vdim=10, conv=2), latent(heads=2, dim=24, rot_dim=16, vdim=8, kv_rank=48, rot_dims=8)],
                              width=40, ff=64, loop=(0, 2, 2), no_mlp=(0,)),
    "no_loop": config([latent(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=96, scale=0.3), windowed(heads=4, dim=8, vdim=8, kv_rank=64, window=7),
                       delta(heads=2, kv_heads=1, dim=64, vdim=32, conv=1)], width=64, vocab=130, ff=128, no_mlp=(2,), logit_softcap=None),
    "loop_once": config([delta(), windowed(heads=1, dim=16, vdim=48, kv_rank=20, window=5)], loop=(1, 2, 1), eps=1e-6, logit_scale=None),
    "only_latent": config([latent(), windowed(heads=5, dim=8, vdim=8, kv_rank=128, window=36)], loop=(0, 2, 2), ff=100),
    "only_delta": config([delta(), delta(heads=6, kv_heads=3, dim=12, vdim=16, conv=2)], loop=(1, 2, 2), logit_scale=1.0, logit_softcap=None),
    # nothing a multiple of 4 or 8: width, feed-forward, heads' sizes, the latent, taps beyond four
    "odd_sizes": config([latent(heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=13, rot_dims=6), delta(heads=3, kv_heads=1, dim=9, vdim=7, conv=5),
                         windowed(heads=2, dim=5, vdim=9, kv_rank=11, window=3)], width=50, vocab=61, ff=45, loop=(1, 3, 2)),
}


def make_model(path: Path, cfg: dict, seed: int = 0, sharp: float = 1.0) -> dict:
    """Writes the folder; returns the tensors as float64 arrays (as stored: values a bfloat16 engine reads unchanged)."""
    arch = resolve_architecture(cfg)
    decls = declared_tensors(arch.model_spec(arch.parse_config(cfg)))
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=g) * std

    def uniform(shape, lo, hi):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    tensors = {}
    for name, decl in sorted(decls.items()):
        if decl.optional_alias_of:
            continue
        shape = tuple(decl.shape)
        if name.endswith("A_log"):
            t = uniform(shape, -5.0, -2.0)  # decays close to one: the state remembers
        elif name.endswith("dt_bias"):
            t = uniform(shape, -2.0, 0.5)
        elif name.endswith(".conv"):
            t = normal(shape, 0.6)
        elif name == "loop.step":
            t = normal(shape, 0.7)
        elif name.endswith("dkv.norm"):
            t = sharp * (1.5 + normal(shape, 0.3))  # sharp attention: single keys matter
        elif name.endswith("mix.norm"):
            t = 1.0 + normal(shape, 0.2)
        elif len(shape) == 1:
            t = normal(shape, 0.2)  # norm weights are stored as the deviation from one
        elif name == "embed":
            t = normal(shape, 1.0)
        else:
            t = normal(shape, 1.0 / shape[1] ** 0.5)
        tensors[name] = t.to(torch.bfloat16).float()
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", tensors)
    return {k: v.double().numpy() for k, v in tensors.items()}


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def rounding_error(path, device, dtype, toks, want):
    """What rounding alone does to this sequence in bfloat16: the error of the whole prompt, alone, in a fresh engine.
    A schedule may not add to it."""
    if dtype == "float32":
        return 0.0
    return float(np.abs(Session(path, device, dtype, pages=len(toks) // 8 + 2).whole("alone", toks) - want).max())


def forward_with_layers(cfg, w, toks):
    trace = []
    return plain.forward(cfg, w, toks, trace), np.stack(trace)


# ----------------------------------------------------------------------------- cases


def case_every_configuration_whole_prompt_and_layers(tmp_path, device, dtype):
    """Whole prompts in every configuration: logits, and the stream after every layer run (in float32)."""
    for name, cfg in CONFIGS.items():
        w = make_model(tmp_path / name, cfg, seed=3)
        toks = tokens_for(cfg, 77, seed=1)  # more than the 64 tokens from which portions take their own convolution kernel
        want, layers = forward_with_layers(cfg, w, toks)
        s = Session(tmp_path / name, device, dtype)
        s.model.trace_layers = []
        got = s.whole("a", toks)
        close(got, want, dtype, name)
        assert len(s.model.trace_layers) == layers.shape[0] == len(plain.layer_runs(cfg)), name
        if dtype == "float32":
            for i, h in enumerate(s.model.trace_layers):
                close(h.double().cpu().numpy(), layers[i], dtype, f"{name}: stream after layer run {i}")
        s.model.trace_layers = None


def case_each_mechanism_alone(tmp_path, device, dtype):
    """One layer, no loop: each mixer with nothing beside it, each mixer's variants, and the feed-forward beside the
    simplest mixer; cache rows of 64 and 128 numbers (which the TMA-fed attention kernels take in bfloat16), of a size
    that is no multiple of 16, and beyond 256."""
    layers = {
        "latent": latent(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=24, scale=0.9),
        "latent_partial_rotation": latent(heads=2, dim=32, rot_dim=24, vdim=8, kv_rank=40, rot_dims=8),
        "latent_row_64": latent(heads=8, dim=16, rot_dim=16, vdim=32, kv_rank=48),
        "latent_row_128": latent(heads=5, dim=24, rot_dim=32, vdim=16, kv_rank=96),
        "latent_row_odd": latent(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=21),
        "latent_row_wide": latent(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=272),
        "windowed": windowed(),
        "windowed_row_64": windowed(heads=4, dim=32, vdim=16, kv_rank=64, window=9),
        "windowed_row_128": windowed(heads=16, dim=8, vdim=8, kv_rank=128, window=30),
        "delta": delta(heads=6, kv_heads=2, dim=12, vdim=10, conv=3),
        "delta_one_tap": delta(heads=1, kv_heads=1, dim=32, vdim=64, conv=1),
        "delta_wide": delta(heads=2, kv_heads=2, dim=136, vdim=40, conv=4),
    }
    for name, layer in layers.items():
        cfg = config([layer], no_mlp=(0,))
        w = make_model(tmp_path / name, cfg, seed=5)
        toks = tokens_for(cfg, 45, seed=2)
        close(Session(tmp_path / name, device, dtype, pages=12).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)
    for name, ff in (("feed_forward_64", 128), ("feed_forward_odd", 52)):
        cfg = config([windowed(heads=1, dim=8, vdim=8, kv_rank=16, window=3)], ff=ff)
        w = make_model(tmp_path / name, cfg, seed=6)
        toks = tokens_for(cfg, 30, seed=3)
        close(Session(tmp_path / name, device, dtype).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)


def case_prefill_then_token_by_token(tmp_path, device, dtype):
    """A prompt in one step, then 60 tokens one at a time (the windows pass over decoded tokens), against the whole
    sequence at once; and a sequence fed token by token from its very first token."""
    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "m", cfg, seed=7)
    toks = tokens_for(cfg, 95, seed=3)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "m", device, dtype, pages=40)
    got = [s.step(("a", toks[:35], list(range(35))))]
    got += [s.step(("a", [t], [0])) for t in toks[35:]]
    close(np.concatenate(got), want, dtype, "prompt then decode", rounding_error(tmp_path / "m", device, dtype, toks, want))
    s.free("a")
    got = [s.step(("b", [t], [0])) for t in toks[:20]]
    close(np.concatenate(got), want[:20], dtype, "token by token from the start")


def case_long_decoding(tmp_path, device, dtype):
    """A short prompt and 300 decoded tokens in a model of delta layers and windows: the state is carried through
    hundreds of steps, pages behind the windows are given back on the way."""
    cfg = config([delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=4), windowed(window=21), latent(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16)],
                 loop=(0, 2, 2), width=32, ff=64)
    w = make_model(tmp_path / "l", cfg, seed=9)
    toks = tokens_for(cfg, 310, seed=4)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "l", device, dtype, pages=44, page_size=8)
    s.step(("a", toks[:10], []))
    got = np.concatenate([s.step(("a", [t], [0])) for t in toks[10:]])
    close(got, want[10:], dtype, "long decoding", rounding_error(tmp_path / "l", device, dtype, toks, want))
    forgot = plain.forward(cfg, w, toks[200:])
    assert np.abs(forgot[-1] - want[-1]).max() > 0.05, "the state does not remember enough for this test"


def case_portions_of_many_sizes(tmp_path, device, dtype):
    """Portions down to two tokens and single tokens between them, cut inside pages and windows and shorter than the
    convolution's reach."""
    for name in ("mixed_loop", "loop_from_start", "no_loop"):
        cfg = CONFIGS[name]
        w = make_model(tmp_path / name, cfg, seed=11)
        toks = tokens_for(cfg, 64, seed=5)
        want = plain.forward(cfg, w, toks)
        s = Session(tmp_path / name, device, dtype)
        got, at = [], 0
        for n in (2, 1, 2, 3, 1, 1, 9, 2, 16, 1, 7, 2, 2, 15):
            got.append(s.step(("a", toks[at : at + n], list(range(n)))))
            at += n
        assert at == 64
        close(np.concatenate(got), want, dtype, name, rounding_error(tmp_path / name, device, dtype, toks, want))


def case_batches_of_unequal_requests(tmp_path, device, dtype):
    """Up to four live requests: portions of some beside single tokens of others; a request sits out a step; the
    logits of each equal those of the request alone."""
    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "m", cfg, seed=13)
    seqs = {r: tokens_for(cfg, n, seed=20 + i) for i, (r, n) in enumerate((("a", 50), ("b", 33), ("c", 9), ("d", 41)))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    s = Session(tmp_path / "m", device, dtype, pages=40)
    at = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}
    plan = [{"a": 17, "b": 2}, {"a": 1, "b": 20, "c": 3}, {"a": 1, "c": 1, "d": 30}, {"b": 1, "c": 1, "d": 1, "a": 9}, {"a": 2, "b": 2, "c": 2, "d": 2},
            {"a": 1, "b": 1, "c": 1, "d": 1}, {"d": 1, "c": 1}, {"a": 19, "b": 7, "d": 7}]
    for step in plan:
        parts = []
        for r, n in step.items():
            n = min(n, len(seqs[r]) - at[r])
            parts.append((r, seqs[r][at[r] : at[r] + n], list(range(n))))
        out = s.step(*parts)
        row = 0
        for r, t, _ in parts:
            got[r].append(out[row : row + len(t)])
            row += len(t)
            at[r] += len(t)
    for r in seqs:
        close(np.concatenate(got[r]), want[r][: at[r]], dtype, f"request {r}", rounding_error(tmp_path / "m", device, dtype, seqs[r], want[r]))


def case_pages_and_slots_used_again(tmp_path, device, dtype):
    """A pool for two short requests and two state slots: request after request takes the pages and the slot a
    finished one gave back, and computes what it would compute in a fresh engine."""
    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "m", cfg, seed=17)
    s = Session(tmp_path / "m", device, dtype, pages=8, page_size=8, max_requests=2)
    seqs = [tokens_for(cfg, n, seed=40 + i) for i, n in enumerate((30, 25, 31, 12, 28))]
    live = []
    for i, toks in enumerate(seqs):
        if len(live) == 2:
            s.free(live.pop(0))
        cut = len(toks) // 2
        a = s.step((i, toks[:cut], list(range(cut))))
        b = s.step((i, toks[cut:], list(range(len(toks) - cut))))
        want = plain.forward(cfg, w, toks)
        close(np.concatenate([a, b]), want, dtype, f"request {i}", rounding_error(tmp_path / "m", device, dtype, toks, want))
        live.append(i)
    s.manager.check_invariants()


def _deciding_pair(cfg, w):
    """In a model of one windowed latent layer (no positions) a score depends on the two tokens alone.  Returns a token
    whose first head gives one other token's key a score far above every other's, that token, and tokens whose keys it
    scores far below."""
    mix, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    h = plain.offset_norm(w["embed"], w["l0.norm1"], eps)
    q = (h @ w["l0.mix.q"].T)[:, : mix["dim"]]
    c = plain.rms_unit(h @ w["l0.mix.dkv"].T, eps) * w["l0.mix.dkv.norm"]
    k = (c @ w["l0.mix.uk"].T)[:, : mix["dim"]]
    scores = (q @ k.T) * mix["scale"]
    V = cfg["vocab"]
    asker = next(t for t in range(V) if scores[t].argmax() != t and np.sort(scores[t])[-1] - np.sort(scores[t])[-2] > 8)
    key = int(scores[asker].argmax())
    noise = [t for t in range(V) if scores[asker, t] < scores[asker, key] - 8 and t != asker]
    assert len(noise) > 20
    return asker, key, noise


def case_one_far_key_decides(tmp_path, device, dtype):
    """Attention over the latent alone (a window wider than the sequence, a large scale), and a sequence made so that
    the last token's first head puts nearly all its mass on ONE key among hundreds — at a page border, beside one, at
    the very start: a kernel that skips or misplaces that key changes the logits by far more than the tolerance.  In
    a prompt portion and decoded."""
    cfg = config([windowed(heads=2, dim=16, vdim=16, kv_rank=24, scale=3.0, window=100000)], width=32, vocab=50, no_mlp=(0,))
    w = make_model(tmp_path / "far", cfg, seed=19)
    asker, key, noise = _deciding_pair(cfg, w)
    s = Session(tmp_path / "far", device, dtype, pages=48, page_size=8)
    for far in (8, 15, 16, 1, 0, 100, 263):
        toks = [noise[i] for i in np.random.default_rng(far).integers(0, len(noise), 330)]
        toks[far] = key
        toks[-1] = asker
        want = plain.forward(cfg, w, toks)
        without = list(toks)
        without[far] = noise[0]
        assert np.abs(plain.forward(cfg, w, without)[-1] - want[-1]).max() > 2.0, "the far key does not matter enough for this test"
        close(s.whole("p", toks)[-1], want[-1], dtype, f"far key {far} in a prompt")
        s.free("p")
        s.step(("d", toks[:-1], []))
        close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"far key {far} decoded")
        s.free("d")


def case_one_key_at_the_window_s_edge(tmp_path, device, dtype):
    """The same construction with a window of 24 keys: the deciding key sits on the last place the window still holds
    (it decides), and one place further back (it must not be seen); in a prompt and decoded alone, with the window's
    edge inside a page and on a page border."""
    window = 24
    cfg = config([windowed(heads=2, dim=16, vdim=16, kv_rank=24, scale=3.0, window=window)], width=32, vocab=50, no_mlp=(0,))
    w = make_model(tmp_path / "edge", cfg, seed=19)
    asker, key, noise = _deciding_pair(cfg, w)
    s = Session(tmp_path / "edge", device, dtype, pages=24, page_size=8)
    for length in (60, 57):  # the oldest visible key at 36 (inside a page) and at 33; its neighbour outside at 35 and 32 (a page's first key)
        last = length - 1
        inside, outside = last - window + 1, last - window
        logits = {}
        for name, place in (("inside", inside), ("outside", outside)):
            toks = [noise[i] for i in np.random.default_rng(length).integers(0, len(noise), length)]
            toks[place] = key
            toks[last] = asker
            want = plain.forward(cfg, w, toks)
            logits[name] = want[-1]
            close(s.whole("p", toks)[-1], want[-1], dtype, f"key {name} the window, prompt of {length}")
            s.free("p")
            s.step(("d", toks[:-1], []))
            close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"key {name} the window, decoded at {last}")
            s.free("d")
            s.step(("c", toks[: last - 5], []))  # the window's edge inside a portion that ends the prompt
            close(s.step(("c", toks[last - 5 :], [5]))[0], want[-1], dtype, f"key {name} the window, in a last portion of 6")
            s.free("c")
        assert np.abs(logits["inside"] - logits["outside"]).max() > 2.0, "the key at the window's edge does not matter enough for this test"


def case_rotation_far_back(tmp_path, device, dtype):
    """The mixer with the rotated key part over 300 tokens, whole and with its last 40 tokens decoded: keys of
    every distance matter, and the angles reach hundreds of radians."""
    cfg = config([latent(heads=2, dim=8, rot_dim=16, vdim=16, kv_rank=16, scale=0.3, base=50.0)], width=32, vocab=60, no_mlp=(0,))
    w = make_model(tmp_path / "rot", cfg, seed=23)
    toks = tokens_for(cfg, 300, seed=6)
    want = plain.forward(cfg, w, toks)
    assert np.abs(plain.forward(cfg, w, toks[100:])[-1] - want[-1]).max() > 0.05, "far keys do not matter enough for this test"
    s = Session(tmp_path / "rot", device, dtype, pages=44, page_size=8)
    rounding = rounding_error(tmp_path / "rot", device, dtype, toks, want)
    got = [s.step(("a", toks[:260], list(range(260))))] + [s.step(("a", [t], [0])) for t in toks[260:]]
    close(np.concatenate(got), want, dtype, "rotation", rounding)


def case_the_first_tokens(tmp_path, device, dtype):
    """Sequences of one, two and three tokens, and a first step of one token followed by a portion: the convolution's
    zeros before the start, a state that starts from zero, windows and pages that are not full."""
    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "m", cfg, seed=27)
    s = Session(tmp_path / "m", device, dtype)
    for n in (1, 2, 3):
        toks = tokens_for(cfg, n, seed=70 + n)
        close(s.whole("a", toks), plain.forward(cfg, w, toks), dtype, f"{n} tokens")
        s.free("a")
    toks = tokens_for(cfg, 12, seed=75)
    got = np.concatenate([s.step(("b", toks[:1], [0])), s.step(("b", toks[1:3], [0, 1])), s.step(("b", toks[3:], list(range(9))))])
    close(got, plain.forward(cfg, w, toks), dtype, "one token, then portions")


def case_the_soft_cap_bends_large_logits(tmp_path, device, dtype):
    """Logits that would reach about twice the cap come out bent into (-cap, cap), and equal to the plain model's."""
    cfg = config([windowed(heads=1, dim=8, vdim=8, kv_rank=16, window=4)], width=32, vocab=40, logit_scale=0.5, logit_softcap=5.0)
    w = make_model(tmp_path / "cap", cfg, seed=29)
    toks = tokens_for(cfg, 9, seed=8)
    want = plain.forward(cfg, w, toks)
    assert 4.5 < np.abs(want).max() < 5.0
    uncapped = json.loads(json.dumps(cfg))
    del uncapped["logit_softcap"]
    assert np.abs(plain.forward(uncapped, w, toks)).max() > 9.0
    close(Session(tmp_path / "cap", device, dtype).whole("a", toks), want, dtype, "soft cap")


def case_layer_sizes_of_a_larger_model(tmp_path, device, dtype):
    """Heads of 128 x 128 in the delta rule and cache rows of 128 numbers (which the TMA-fed and tcgen05 attention kernels
    take in bfloat16, with several tiles of queries and keys), a prompt of 300 tokens in two portions, then decoding."""
    cfg = config([windowed(heads=8, dim=64, vdim=64, kv_rank=128, scale=0.2, window=150), delta(heads=4, kv_heads=2, dim=128, vdim=128, conv=4),
                  latent(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=0.2)], width=256, vocab=300, ff=512, loop=(0, 2, 2))
    w = make_model(tmp_path / "big", cfg, seed=37)
    toks = tokens_for(cfg, 320, seed=12)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "big", device, dtype, pages=48, page_size=16)
    rows = [0, 1, 15, 16, 127, 128, 129, 149, 150, 151, 199]
    got = [s.step(("a", toks[:200], rows)), s.step(("a", toks[200:300], list(range(100))))]
    got += [s.step(("a", [t], [0])) for t in toks[300:]]
    rounding = rounding_error(tmp_path / "big", device, dtype, toks, want)
    close(np.concatenate(got), np.concatenate([want[rows], want[200:]]), dtype, "larger sizes", rounding)


def case_greedy_generation_through_the_engine(tmp_path, device, dtype):
    """LLMEngine.generate (scheduler, batching, sampler) against greedy decoding with the plain model."""
    from dli_b200 import LLMEngine, SamplingParams, SchedulerConfig

    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "g", cfg, seed=31)
    prompts = [tokens_for(cfg, n, seed=60 + n) for n in (5, 19, 1, 11, 8)]
    if device == "cpu":
        from tests import cpu_ops

        model = dli_b200.load_model(tmp_path / "g", dtype, device)
        runner = ModelRunner(model, num_pages=32, page_size=8, max_requests=4, cuda_graphs=False)
        engine = LLMEngine(runner, SchedulerConfig(4, 24), sampler=cpu_ops.CpuSampler())
    else:
        engine = LLMEngine.from_model_dir(tmp_path / "g", dtype=dtype, device=device, num_blocks=32, block_size=8, config=SchedulerConfig(4, 24))
    outs = engine.generate(prompts, SamplingParams(max_tokens=10))
    tol = TOL[dtype]
    compared = 0
    for p, got in zip(prompts, outs):
        toks = list(p)
        for t in got:
            row = plain.forward(cfg, w, toks)[-1]
            top = np.sort(row)[-2:]
            if int(np.argmax(row)) != t:
                assert top[1] - top[0] < 2 * tol * max(1.0, np.abs(row).max()), "a generated token differs from the plain model's"
                break
            toks.append(t)
            compared += 1
    assert compared >= 25


CASES = [v for k, v in sorted(globals().items()) if k.startswith("case_")]
