"""The Pazenex model through the engine's host side on the CPU (float32, torch stand-ins for the kernels) against the
plain implementation; configuration parsing and run order.  The GPU tests run the same cases on the real kernels."""

import json

import pytest

from dli_b200.config.pazenex import PazenexConfig, pazenex_run_order
from dli_b200.config.llama import UnsupportedModelError
from dli_b200.config.registry import resolve_architecture
from tests import cpu_ops, pazenex_suite as suite
from tests.plain import pazenex_plain as plain


@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, tmp_path):
    with cpu_ops.patched():
        case(tmp_path, "cpu", "float32")


def test_run_order_follows_the_loop():
    for name, cfg in suite.CONFIGS.items():
        parsed = resolve_architecture(cfg).parse_config(cfg)
        order = pazenex_run_order(parsed)
        start = (cfg.get("loop") or {}).get("start")
        assert [(s.layer, s.entry) for s in order] == [(i, t if i == start else None) for i, t in plain.layer_runs(cfg)], name
        assert all(s.cache_of is None for s in order)  # every pass keeps a cache and a state of its own


def test_configuration_is_read_strictly():
    good = suite.CONFIGS["mixed_loop"]
    assert isinstance(PazenexConfig.from_dict(good), PazenexConfig)
    for path, value in ((("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "vdim"), 8), (("layers", 0, "mixer", "rot", "dims"), 7),
                        (("layers", 1, "mixer", "groups"), 3), (("layers", 1, "mixer", "norm_groups"), 5), (("layers", 0, "type"), "other"),
                        (("loop", "stop"), 9), (("loop", "times"), 0), (("layers", 0, "mlp", "kind"), "routed")):
        bad = json.loads(json.dumps(good))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            PazenexConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    bad["layers"][1]["mixer"]["surprise"] = 1
    with pytest.raises(UnsupportedModelError):
        PazenexConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][1]["mixer"]["state"]
    with pytest.raises(KeyError):
        PazenexConfig.from_dict(bad)
