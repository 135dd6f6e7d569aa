"""Autotuner components one by one: shape buckets, configuration spaces, the configuration cache (age and device
filters, atomic save), each search strategy on a synthetic cost surface, and AutoTuner's cache / improvement logic with
a host-timed kernel (the unit tests of crates/autotuner/src/{kernel_config,cache,search,tuner}.rs)."""
import json
import time

import pytest

from rustral_b200.tune import (AutoTuner, BayesianSearch, ConfigCache, ConfigSpace, EvolutionarySearch, GridSearch,
                               MatmulShapeBucket, PerfMetrics, RandomSearch, Strategy, TunableKernel, TunerConfig, TuningResult,
                               TuningSession, dim_bucket)


def test_dimension_buckets_and_matmul_cache_key():
    assert [dim_bucket(n) for n in (1, 255, 256, 512, 513, 2047, 2048, 8191, 8192)] == \
        ["tiny", "tiny", "small", "small", "medium", "medium", "large", "large", "xlarge"]
    assert MatmulShapeBucket.of(128, 1024, 8192).cache_key() == "matmul_tiny_medium_xlarge"
    assert MatmulShapeBucket.of(300, 300, 300) == MatmulShapeBucket.of(512, 256, 400)


def test_config_space_sizes():
    assert ConfigSpace({"a": [1, 2, 3], "b": [4, 5]}).size() == 6
    assert ConfigSpace.matmul_full().size() == 4 * 6 * 3 and ConfigSpace.matmul_reduced().size() < ConfigSpace.matmul_full().size()


def test_perf_metrics_from_duration():
    m = PerfMetrics.from_duration(500.0, flops=1e12, bytes_=2e9)
    assert m.tflops == pytest.approx(2000.0) and m.gbytes_per_s == pytest.approx(4000.0)
    assert PerfMetrics.from_duration(0.0, 1.0, 1.0).tflops == 0.0


def test_cache_round_trip_hit_rate_and_filters(tmp_path):
    path = str(tmp_path / "sub" / "configs.json")
    c = ConfigCache(path, device_id="B200")
    assert c.get_config("gemm", "B200", "bf16", "matmul_tiny_tiny_tiny") is None
    c.store_config("gemm", "B200", "bf16", "matmul_tiny_tiny_tiny", {"block_n": 128}, 12.5, 7)
    c.store_config("gemm", "H100", "bf16", "matmul_tiny_tiny_tiny", {"block_n": 64}, 20.0, 3)
    e = c.get_config("gemm", "B200", "bf16", "matmul_tiny_tiny_tiny")
    assert e.config == {"block_n": 128} and e.time_us == 12.5 and e.num_samples == 7 and c.hit_rate() == 0.5
    c.save()
    raw = json.load(open(path))
    assert set(raw) == {ConfigCache.key("gemm", "B200", "bf16", "matmul_tiny_tiny_tiny"), ConfigCache.key("gemm", "H100", "bf16", "matmul_tiny_tiny_tiny")}
    again = ConfigCache(path, device_id="B200")                               # the other device's entry is ignored on load
    assert list(again.entries) == [ConfigCache.key("gemm", "B200", "bf16", "matmul_tiny_tiny_tiny")]
    stale = dict(raw)
    for v in stale.values():
        v["timestamp"] = time.time() - ConfigCache.MAX_AGE_S - 10
    json.dump(stale, open(path, "w"))
    assert ConfigCache(path, device_id="B200").entries == {}                  # older than 30 days
    open(path, "w").write("{not json")
    assert ConfigCache(path).entries == {}                                    # a corrupt file is an empty cache, not an error


def _cost(c):
    return 10.0 + abs(c["x"] - 6) * 2.0 + abs(c["y"] - 2) * 5.0


@pytest.mark.parametrize("cls,budget", [(GridSearch, 0), (RandomSearch, 40), (EvolutionarySearch, 40), (BayesianSearch, 30)])
def test_search_strategies_find_the_minimum_of_a_separable_surface(cls, budget):
    space = ConfigSpace({"x": list(range(10)), "y": [0, 1, 2, 3]})
    s = cls(space, seed=3, max_evals=budget)
    seen = set()
    while True:
        c = s.next_config()
        if c is None:
            break
        assert set(c) == {"x", "y"} and c["x"] in space.dims["x"] and c["y"] in space.dims["y"]
        seen.add((c["x"], c["y"]))
        s.report(c, _cost(c))
    best, t = s.best()
    if cls is GridSearch:
        assert len(seen) == 40 and s.num_evals() == 40                         # the grid visits every point once
    else:
        assert s.num_evals() <= budget
    # the heuristics get within one step of the optimum in their budget; grid and the model-based search find it exactly
    assert t == _cost(best) and t <= 14.0 and (cls in (RandomSearch, EvolutionarySearch) or best == {"x": 6, "y": 2})


def test_search_is_reproducible_for_a_seed():
    space = ConfigSpace({"x": list(range(10)), "y": [0, 1, 2, 3]})
    runs = []
    for _ in range(2):
        s = RandomSearch(space, seed=11, max_evals=8)
        runs.append([tuple(sorted(s.next_config().items())) for _ in range(8)])
    assert runs[0] == runs[1] and RandomSearch(space, seed=12, max_evals=8).next_config() is not None


def test_tuning_session_records_trials_and_reports_the_best():
    sess = TuningSession("gemm", "m128")
    for c, t in (({"a": 1}, 9.0), ({"a": 2}, 4.0), ({"a": 3}, 6.0)):
        sess.record(c, t)
    sess.finish()
    d = sess.to_dict()
    assert sess.best == ({"a": 2}, 4.0) and d["best_config"] == {"a": 2} and d["best_time_us"] == 4.0 and d["num_trials"] == 3
    assert sess.finished_at >= sess.started_at and d["elapsed_s"] >= 0 and TuningSession("k", "s").best == (None, float("inf"))


class _SleepKernel(TunableKernel):
    """A kernel whose cost is a table lookup, timed on the host."""
    kernel_id = "sleep"
    host_timed = True

    def __init__(self, table):
        self.table, self.calls = table, []

    def config_space(self):
        return ConfigSpace({"v": list(self.table)})

    def with_config(self, config):
        def run():
            self.calls.append(config["v"])
            time.sleep(self.table[config["v"]])
        return run

    def input_signature(self):
        return "sig"


def test_autotuner_picks_the_fastest_config_caches_it_and_reuses_the_cache(tmp_path):
    cache = ConfigCache(str(tmp_path / "c.json"), device_id="dev")
    cfg = TunerConfig(Strategy.GRID, warmup=0, timing=1, max_evals=8, device_id="dev", min_improvement_pct=5.0)
    k = _SleepKernel({0: 0.004, 1: 0.0005, 2: 0.003})
    res = AutoTuner(cfg, cache).tune(k)
    assert isinstance(res, TuningResult) and res.config == {"v": 1} and not res.from_cache and res.improvement_pct > 50
    assert cache.get_config("sleep", "dev", "bf16", "sig").config == {"v": 1}
    k2 = _SleepKernel({0: 0.004, 1: 0.0005, 2: 0.003})
    tuner = AutoTuner(cfg, ConfigCache(str(tmp_path / "c.json"), device_id="dev"))
    res2 = tuner.tune(k2)
    assert res2.from_cache and res2.config == {"v": 1} and set(k2.calls) == {1} and tuner.stats["cache_hits"] == 1


def test_autotuner_keeps_the_default_when_the_gain_is_below_the_threshold_and_when_disabled(tmp_path):
    cfg = TunerConfig(Strategy.GRID, warmup=0, timing=1, max_evals=4, device_id="dev", min_improvement_pct=90.0, use_cache=False,
                      cache_results=False)
    k = _SleepKernel({0: 0.002, 1: 0.0015})
    assert AutoTuner(cfg, ConfigCache(str(tmp_path / "x.json"))).tune(k).config == {"v": 0}
    off = AutoTuner(TunerConfig.disabled(), ConfigCache(str(tmp_path / "y.json")))
    k3 = _SleepKernel({0: 0.001, 1: 0.0001})
    r = off.tune(k3)
    assert r.config == {"v": 0} and r.evaluated == 0 and k3.calls == []
    ci = TunerConfig.ci_safe()
    assert ci.ci_mode and ci.max_evals <= 5 and TunerConfig.fast().max_tuning_time_s <= TunerConfig().max_tuning_time_s


def test_command_line_cache_and_shapes(tmp_path, monkeypatch, capsys):
    from rustral_b200.tune import ConfigCache
    from rustral_b200.tune.__main__ import main
    monkeypatch.setenv("RUSTRAL_CACHE_DIR", str(tmp_path))
    c = ConfigCache()
    c.store_config("gemm_bf16_tcgen05", "B200", "bf16", "matmul_large_large_medium", {"block_n": 256}, 12.5, 8)
    c.save()
    assert main(["cache"]) == 0
    out = capsys.readouterr().out
    assert "total entries: 1" in out and "B200: 1" in out
    assert main(["cache", "--json"]) == 0
    assert '"block_n": 256' in capsys.readouterr().out
    assert main(["shapes", "--model", "gpt2-small", "--tokens", "4096"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 5 and lines[0].startswith("4096 x 2304 x 768") and "matmul_large_large_medium" in lines[0]
    assert main(["cache", "--clear"]) == 0 and ConfigCache().entries == {}
