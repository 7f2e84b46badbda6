"""Host-side decisions that need no GPU: when uncached rows are staged, and how bench.py turns the library's event
totals into the roofline object."""
import importlib.util
import os
import sys

import pytest

from neutronbench_b200.toolkit import GCNConfig, default_stage_misses

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(**kw):
    base = dict(layers=[16, 8, 4], fanout=(5, 5), batch_size=64)
    base.update(kw)
    return GCNConfig(**base)


@pytest.mark.parametrize("kw,sharded,on_device,world,expect", [
    (dict(), False, True, 1, False),                                   # table in HBM: nothing to stage
    (dict(), False, False, 1, False),                                  # host table, one rank: read in place
    (dict(), False, False, 4, True),                                   # host table shared by several ranks
    (dict(cache_type="rate", cache_rate=1.0), False, False, 8, False), # everything cached: no misses
    (dict(cache_type="rate", cache_rate=0.2), False, False, 2, True),
    (dict(), True, False, 1, True),                                    # a sharded table is read through staging
    (dict(stage_misses=False), False, False, 8, False),                # an explicit setting wins
    (dict(stage_misses=True), False, True, 1, True),
])
def test_default_stage_misses(kw, sharded, on_device, world, expect):
    assert default_stage_misses(_cfg(**kw), sharded, on_device, world) is expect


def _bench():
    spec = importlib.util.spec_from_file_location("nb_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nb_bench"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_roofline_from_the_library_event_totals():
    """`roofline` is the dominant kernel's bytes over its event time from the timed regions; `all_aggregation` every
    class of the fully timed region that follows them."""
    bench = _bench()
    cfg = _cfg()
    events = ("engine", (0.065 * 20, 247_000_000 * 20, 20), [0.065 * 20, 0.018 * 20], [247_000_000 * 20, 15_800_000 * 20],
              [20, 20])
    roof, all_agg = bench.roofline_of(events, 6551.4, "measured", 272_000_000, cfg)
    assert roof["launches"] == 20 and abs(roof["avg_launch_ms"] - 0.065) < 1e-12
    assert abs(roof["achieved"] - 247_000_000 / 0.065e-3 / 1e9) < 1e-6          # 3800 GB/s
    assert abs(roof["frac"] - roof["achieved"] / 6551.4) < 1e-12 and roof["traffic"] == 272_000_000
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s"
    total_b, total_ms = (247_000_000 + 15_800_000) * 20, (0.065 + 0.018) * 20
    assert abs(all_agg["achieved"] - total_b / (total_ms * 1e-3) / 1e9) < 1e-6 and all_agg["launches"] == 40
