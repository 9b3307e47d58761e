"""The Sugonex model through the engine's host side on the CPU (float32, torch stand-ins for the kernels) against the
plain implementation; configuration parsing and run order.  The GPU tests run the same cases on the real kernels."""

import json
import warnings

import pytest

from dli_b200.config.llama import UnsupportedModelError
from dli_b200.config.registry import resolve_architecture
from dli_b200.config.sugonex import SugonexConfig, sugonex_run_order
from tests import cpu_ops, sugonex_suite as suite
from tests.plain import sugonex_plain as plain


@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, tmp_path):
    with cpu_ops.patched():
        case(tmp_path, "cpu", "float32")


def test_run_order_follows_the_loop():
    for name, cfg in suite.CONFIGS.items():
        parsed = resolve_architecture(cfg).parse_config(cfg)
        order = sugonex_run_order(parsed)
        start = (cfg.get("loop") or {}).get("start")
        assert [(s.layer, s.entry) for s in order] == [(i, t if i == start else None) for i, t in plain.layer_runs(cfg)], name
        assert all(s.cache_of is None for s in order)  # every pass keeps a cache and a state of its own


def test_configuration_is_checked():
    good = suite.CONFIGS["mixed_loop"]
    parsed = SugonexConfig.from_dict(good)
    assert isinstance(parsed, SugonexConfig) and parsed.logit_scale == good["logit_scale"] and parsed.logit_softcap == good["logit_softcap"]
    assert parsed.layers[0].mixer.window == 13 and not parsed.layers[0].mixer.gate and parsed.layers[2].mixer.gate
    for path, value in ((("layers", 1, "mixer", "kv_heads"), 3), (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 2, "mixer", "rot", "dims"), 10),
                        (("layers", 0, "type"), "other"), (("loop", "stop"), 9), (("loop", "times"), 0), (("layers", 0, "mlp", "kind"), "routed"),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("logit_softcap",), -1.0), (("layers", 1, "mixer", "conv"), 0)):
        bad = json.loads(json.dumps(good))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            SugonexConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][1]["mixer"]["conv"]
    with pytest.raises(KeyError):
        SugonexConfig.from_dict(bad)
    extra = json.loads(json.dumps(good))
    extra["layers"][1]["mixer"]["surprise"] = 1
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        assert SugonexConfig.from_dict(extra) == parsed  # a key the parser does not know is reported, not obeyed
    assert any("surprise" in str(w.message) for w in seen)
    plainer = json.loads(json.dumps(good))
    del plainer["logit_scale"], plainer["logit_softcap"], plainer["loop"]
    parsed = SugonexConfig.from_dict(plainer)
    assert parsed.logit_scale == 1.0 and parsed.logit_softcap is None and parsed.loop is None
