"""Cases that compare the engine's Pazenex model with the plain implementation (tests/plain/pazenex_plain.py).

Each case takes (tmp_path, device, dtype) and builds its own small configuration and weights.  The CPU tests
run them on torch stand-ins for the kernels (float32), the GPU tests on the real kernels in both dtypes.
Weights are drawn so that faults show: slow decays (a lost state changes later tokens), sharp attention
(one missing key changes the logits), convolution taps, skips and loop vectors of order one.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import dli_b200
from dli_b200.config.registry import resolve_architecture
from dli_b200.engine import ModelRunner, StepEntry
from dli_b200.parts.model import declared_tensors
from dli_b200.weights import write_safetensors
from tests.plain import pazenex_plain as plain

TOL = {"float32": 3e-4, "bfloat16": 8e-2}


def attention(heads=4, kv_heads=2, dim=16, rot_dims=8, base=10000.0, factor=2.0, scale=0.7, **more):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot, **more}}


def mamba(heads=4, vdim=8, state=8, groups=2, conv=4, norm_groups=4):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def config(layers, width=48, vocab=97, ff=80, loop=None, eps=1e-5, no_mlp=()):
    out = {"architecture": "Pazenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for i, layer in enumerate(layers):
        out["layers"].append({**layer, "mlp": None if i in no_mlp else {"kind": "dense", "ff": ff}})
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# sizes that differ from one another in every respect: head counts and groups, partial and full rotation, odd state
# and head sizes, tap counts from 1 to 4, norm parts, loops from the first layer, over everything, once, or absent
CONFIGS = {
    "mixed_loop": config([attention(), mamba(), attention(heads=6, kv_heads=6, dim=8, rot_dims=8, factor=None, scale=1.1), mamba(conv=2, norm_groups=1)],
                         loop=(1, 3, 3)),
    "loop_from_start": config([mamba(heads=3, vdim=20, state=10, groups=3, conv=3, norm_groups=5), attention(heads=3, kv_heads=1, dim=32, rot_dims=32)],
                              width=40, loop=(0, 2, 2), no_mlp=(0,)),
    "no_loop": config([attention(heads=2, kv_heads=1, dim=64, rot_dims=16, scale=0.4), mamba(heads=2, vdim=16, state=32, groups=1, conv=1, norm_groups=2)],
                      width=64, vocab=130, no_mlp=(1,)),
    "loop_once": config([mamba(), attention(heads=8, kv_heads=2, dim=16, rot_dims=0, factor=None)], loop=(1, 2, 1), eps=1e-6),
    "only_attention": config([attention(), attention(heads=2, kv_heads=2, dim=48, rot_dims=24)], loop=(0, 1, 2)),
    "only_mamba": config([mamba(), mamba(heads=2, vdim=24, state=16, groups=2, conv=2, norm_groups=3)], loop=(1, 2, 2)),
}


def make_model(path: Path, cfg: dict, seed: int = 0) -> dict:
    """Writes the folder; returns the tensors as float64 arrays (as stored: float32 values)."""
    arch = resolve_architecture(cfg)
    decls = declared_tensors(arch.model_spec(arch.parse_config(cfg)))
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=g) * std

    def uniform(shape, lo, hi):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    tensors = {}
    for name, decl in sorted(decls.items()):
        shape = tuple(decl.shape)
        if name.endswith("A_log"):
            t = uniform(shape, -4.0, -1.0)  # decays close to one: the state remembers
        elif name.endswith("dt_bias"):
            t = uniform(shape, -2.0, 0.5)
        elif name.endswith(".D"):
            t = normal(shape, 1.0)
        elif name.endswith("conv"):
            t = normal(shape, 0.6)
        elif name.endswith("conv.b"):
            t = normal(shape, 0.3)
        elif name == "loop.step":
            t = normal(shape, 0.7)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.5 + normal(shape, 0.3)  # sharp attention: single keys matter
        elif len(shape) == 1:
            t = 1.0 + normal(shape, 0.2)
        elif name in ("embed", "head"):
            t = normal(shape, 1.0 if name == "embed" else 0.2)
        else:
            t = normal(shape, 1.5 / shape[1] ** 0.5)
        tensors[name] = t.to(torch.bfloat16).float()  # values a bfloat16 engine reads unchanged
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", tensors)
    return {k: v.double().numpy() for k, v in tensors.items()}


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


class Session:
    """A runner and the bookkeeping a caller does around ``step``."""

    def __init__(self, path, device, dtype, pages=24, page_size=8, max_requests=4, cuda_graphs=True):
        self.model = dli_b200.load_model(path, dtype, device)
        self.runner = ModelRunner(self.model, num_pages=pages, page_size=page_size, max_requests=max_requests, enable_prefix_caching=False,
                                  watermark=0.0, cuda_graphs=cuda_graphs)
        self.manager = self.runner.manager

    def step(self, *parts):
        """parts: (request id, tokens, want).  Returns the wanted logits, in order, as a float64 array."""
        entries = []
        for rid, toks, want in parts:
            if self.manager.has_request(rid):
                self.manager.append_slots(rid, toks)
            else:
                alloc = self.manager.allocate(rid, toks, respect_watermark=False)
                self.runner.start_request(rid, alloc.state_slot)
            entries.append(StepEntry(rid, toks, want))
        out = self.runner.step(entries)
        return out.double().cpu().numpy()

    def whole(self, rid, toks):
        return self.step((rid, toks, list(range(len(toks)))))

    def free(self, rid):
        self.manager.free(rid)


def close(got, want, dtype, what="", rounding=0.0):
    """``rounding``: the error that rounding alone causes on this sequence (``rounding_error``), if the caller measured it:
    three times that is allowed where it exceeds the fixed tolerance."""
    err = np.abs(got - want).max()
    scale = max(1.0, np.abs(want).max())
    assert err <= max(TOL[dtype] * scale, 3 * rounding), f"{what}: max error {err:.3g} (logits up to {scale:.3g}, rounding {rounding:.3g})"


def rounding_error(path, device, dtype, toks, want):
    """What rounding alone does to this sequence in bfloat16: the error of the whole prompt, alone, in a fresh engine.
    The weights of these tests amplify it (sharp attention, long memory); a schedule may not add to it."""
    if dtype == "float32":
        return 0.0
    return float(np.abs(Session(path, device, dtype).whole("alone", toks) - want).max())


# ----------------------------------------------------------------------------- cases


def case_every_configuration_whole_prompt_and_layers(tmp_path, device, dtype):
    """Whole prompts in every configuration: logits, and the stream after every layer run (in float32)."""
    for name, cfg in CONFIGS.items():
        w = make_model(tmp_path / name, cfg, seed=3)
        toks = tokens_for(cfg, 77, seed=1)  # more than the 64 tokens from which portions take their own convolution kernel
        want, layers = plain.forward(cfg, w, toks, return_layers=True)
        s = Session(tmp_path / name, device, dtype)
        s.model.trace_layers = []
        got = s.whole("a", toks)
        close(got, want, dtype, name)
        assert len(s.model.trace_layers) == layers.shape[0], name
        if dtype == "float32":
            for i, h in enumerate(s.model.trace_layers):
                close(h.double().cpu().numpy(), layers[i], dtype, f"{name}: stream after layer run {i}")
        s.model.trace_layers = None


def case_each_mixer_alone(tmp_path, device, dtype):
    """One layer, no feed-forward, no loop: the mixer between its two norms and nothing else."""
    for name, layer in (("attention", attention(heads=4, kv_heads=1, dim=16, rot_dims=16, factor=8.0, scale=0.9)),
                        ("attention_partial_rotation", attention(heads=2, kv_heads=2, dim=32, rot_dims=8, factor=None)),
                        ("mamba", mamba(heads=6, vdim=8, state=12, groups=3, conv=3, norm_groups=2))):
        cfg = config([layer], no_mlp=(0,))
        w = make_model(tmp_path / name, cfg, seed=5)
        toks = tokens_for(cfg, 21, seed=2)
        close(Session(tmp_path / name, device, dtype).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)


def case_prefill_then_token_by_token(tmp_path, device, dtype):
    """A prompt in one step, then 40 tokens one at a time, against the whole sequence at once; and a sequence fed
    token by token from its very first token."""
    cfg = CONFIGS["mixed_loop"]
    w = make_model(tmp_path / "m", cfg, seed=7)
    toks = tokens_for(cfg, 75, seed=3)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "m", device, dtype)
    got = [s.step(("a", toks[:35], list(range(35))))]
    got += [s.step(("a", [t], [0])) for t in toks[35:]]
    close(np.concatenate(got), want, dtype, "prompt then decode")
    s.free("a")
    got = [s.step(("b", [t], [0])) for t in toks[:20]]
    close(np.concatenate(got), want[:20], dtype, "token by token from the start")


def case_portions_of_many_sizes(tmp_path, device, dtype):
    """Portions down to two tokens and single tokens between them, cut inside pages and shorter than the
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
        close(np.concatenate(got), want, dtype, name)


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
        # the other live request decodes between this one's portions
        b = s.step((i, toks[cut:], list(range(len(toks) - cut))))
        want = plain.forward(cfg, w, toks)
        close(np.concatenate([a, b]), want, dtype, f"request {i}", rounding_error(tmp_path / "m", device, dtype, toks, want))
        live.append(i)
    s.manager.check_invariants()


def case_one_far_key_decides(tmp_path, device, dtype):
    """Attention alone (no rotation, a large scale), and a sequence made so that the last token's first head puts
    nearly all its mass on ONE key far back — at a page border, beside one, at the very start: a kernel that skips
    or misplaces that key changes the logits by far more than the tolerance.  In a prompt portion and decoded."""
    cfg = config([attention(heads=2, kv_heads=1, dim=16, rot_dims=0, factor=None, scale=3.0)], width=32, vocab=50, no_mlp=(0,))
    eps, page = cfg["norm"]["eps"], 8
    w = make_model(tmp_path / "far", cfg, seed=19)
    # without rotation a score depends on the two tokens alone: the score of every token's key for every token's query
    h = plain.layer_norm(w["embed"], w["l0.norm1"], eps)
    q = (plain.rms_unit(h @ w["l0.mix.q"].T, eps) * w["l0.mix.q.norm"])[:, :16]
    k = plain.rms_unit(h @ w["l0.mix.k"].T, eps) * w["l0.mix.k.norm"]
    scores = (q @ k.T) * cfg["layers"][0]["mixer"]["scale"]
    asker = next(t for t in range(50) if scores[t].argmax() != t and np.sort(scores[t])[-1] - np.sort(scores[t])[-2] > 8)
    key = int(scores[asker].argmax())
    noise = [t for t in range(50) if scores[asker, t] < scores[asker, key] - 8 and t != asker]
    assert len(noise) > 20
    s = Session(tmp_path / "far", device, dtype, pages=24, page_size=page)
    for far in (8, 15, 16, 1, 0, 100):
        toks = [noise[i] for i in np.random.default_rng(far).integers(0, len(noise), 150)]
        toks[far] = key
        toks[-1] = asker
        want = plain.forward(cfg, w, toks)
        without = list(toks)
        without[far] = noise[0]
        assert np.abs(plain.forward(cfg, w, without)[-1] - want[-1]).max() > 0.2, "the far key does not matter enough for this test"
        close(s.whole("p", toks)[-1], want[-1], dtype, f"far key {far} in a prompt")
        s.free("p")
        s.step(("d", toks[:-1], []))
        close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"far key {far} decoded")
        s.free("d")


def case_the_sink_takes_mass(tmp_path, device, dtype):
    """With every score very negative the sink takes nearly all the mass and the mixer's output vanishes; with a
    softmax without the sink it would not: the first token's output is then the norm of its own value."""
    cfg = config([attention(heads=2, kv_heads=2, dim=8, rot_dims=0, factor=None, scale=-6.0)], width=16, vocab=20, no_mlp=(0,))
    w = make_model(tmp_path / "s", cfg, seed=23)
    # every token is the same, so q . k > 0 at every pair and, with the negative scale, every score is far below the sink's 0
    toks = [5] * 12
    want = plain.forward(cfg, w, toks)
    close(Session(tmp_path / "s", device, dtype).whole("a", toks), want, dtype, "sink")
    cfg_pos = json.loads(json.dumps(cfg))
    cfg_pos["layers"][0]["mixer"]["scale"] = 6.0
    assert np.abs(plain.forward(cfg_pos, w, toks) - want).max() > 0.05


def case_window(tmp_path, device, dtype):
    """The optional window of the attention mixer: keys just inside and just outside it, in a prompt and decoded."""
    cfg = config([attention(heads=2, kv_heads=1, dim=16, rot_dims=8, scale=1.5, window=11), mamba()], loop=(0, 2, 2))
    w = make_model(tmp_path / "w", cfg, seed=29)
    toks = tokens_for(cfg, 40, seed=9)
    want = plain.forward(cfg, w, toks)
    unlimited = json.loads(json.dumps(cfg))
    del unlimited["layers"][0]["mixer"]["window"]
    full = plain.forward(unlimited, w, toks)
    assert np.abs(full[20:] - want[20:]).max() > 0.05
    s = Session(tmp_path / "w", device, dtype, pages=12, page_size=8)
    got = [s.step(("a", toks[:25], list(range(25))))] + [s.step(("a", [t], [0])) for t in toks[25:]]
    close(np.concatenate(got), want, dtype, "window")


def case_one_key_at_the_window_s_edge(tmp_path, device, dtype):
    """The far-key construction with a window of 24 keys: the deciding key sits on the last place the window still
    holds (it decides), and one place further back (it must not be seen); in a prompt and decoded alone, with the
    window's edge inside a page and on a page border."""
    window = 24
    cfg = config([attention(heads=2, kv_heads=1, dim=16, rot_dims=0, factor=None, scale=3.0, window=window)], width=32, vocab=50, no_mlp=(0,))
    eps = cfg["norm"]["eps"]
    w = make_model(tmp_path / "edge", cfg, seed=19)
    h = plain.layer_norm(w["embed"], w["l0.norm1"], eps)
    q = (plain.rms_unit(h @ w["l0.mix.q"].T, eps) * w["l0.mix.q.norm"])[:, :16]
    k = plain.rms_unit(h @ w["l0.mix.k"].T, eps) * w["l0.mix.k.norm"]
    scores = (q @ k.T) * cfg["layers"][0]["mixer"]["scale"]
    asker = next(t for t in range(50) if scores[t].argmax() != t and np.sort(scores[t])[-1] - np.sort(scores[t])[-2] > 8)
    key = int(scores[asker].argmax())
    noise = [t for t in range(50) if scores[asker, t] < scores[asker, key] - 8 and t != asker]
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
        assert np.abs(logits["inside"] - logits["outside"]).max() > 0.2, "the key at the window's edge does not matter enough for this test"


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
