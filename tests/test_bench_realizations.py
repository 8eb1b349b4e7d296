"""bench.py times one realization and its parity pre-flight (tests/headline.py) checks one: they must be the
same dictionary, for every weight form and declared order the benchmark offers. No GPU."""
import importlib.util
import pathlib

import numpy as np
import pytest

import headline


@pytest.fixture(scope="module")
def bench():
    path = pathlib.Path(__file__).resolve().parents[1] / "bench.py"
    spec = importlib.util.spec_from_file_location("bench_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_the_timed_realization_is_the_checked_one(bench):
    paths = list(bench.param_shapes(dict(V=64, D=64, H=4, G=2, FF=96, L=2)))
    scales = {site: 0.01 * (i + 1) for i, site in enumerate(headline.W8A8_SCALED_SITES + (headline.W8A8_ATTN_OUT_SITE,))}
    for attention in ("blockwise", "online", "unfused"):
        for launches in ("merged", "reference"):
            order = {"kind": "device", "attention": attention, "launches": launches}
            for int8, weights in ((False, "bf16"), (True, "int8"), ("e4m3fn", "e4m3fn")):
                assert bench.realization(paths, int8, attention, launches) == headline.realization(paths, order, weights), (attention, launches, weights)
            codes = bench.w8a8_attention_in_codes(attention, launches)
            assert codes == (attention == "online" and launches == "merged")
            assert bench.w8a8_realization(paths, attention, launches, scales) == headline.w8a8_realization(paths, order, scales, attn_out=codes), (attention, launches)
    full = bench.w8a8_realization(paths, "online", "merged", scales)
    assert set(full["scaled"]) == {"RMSNorm.apply/%10", "SwiGLU.apply/%7", "Attention.apply/%22"}
    assert "Attention.apply/%26" in full["accum"] and full["accum"] == full["product"]
    assert all(v["scale"] == float(np.float32(scales[k])) for k, v in full["scaled"].items())


def test_every_workload_names_a_known_kind(bench):
    for name, w in bench.WORKLOADS.items():
        assert w.get("int8", False) in (False, True, "e4m3fn", "w8a8"), name
        if name in bench.GEMM_TRAFFIC:
            assert w.get("kind", "llama") == "llama" and w["B"] * w["T"] == 16384, name
