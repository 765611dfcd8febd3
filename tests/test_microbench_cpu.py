"""The microbenchmark suite on CPU at toy sizes: every numerics experiment runs end to end (run -> JSON -> plot tables),
the timing experiments exercise their plumbing, and the associative-memory engine obeys its invariants."""

import json
import math
import os

import pytest
import torch

from microbench import assoc_mem as am
from microbench import bench_utils as bu
from microbench import plot_style as ps


def test_stats_and_quality_helpers():
    assert bu.stats([]) == (0.0, 0.0, 0.0)
    assert bu.stats([3.0]) == (3.0, 3.0, 3.0)
    med, p25, p75 = bu.stats([1, 2, 3, 4, 5])
    assert (med, p25, p75) == (3.0, 2.0, 4.0)
    m, s = bu.mean_std([1.0, 3.0])
    assert m == 2.0 and abs(s - math.sqrt(2.0)) < 1e-12
    x = torch.randn(3, 16, 24, generator=torch.Generator().manual_seed(0))
    p = bu.polar_factor(x)
    assert torch.allclose(p @ p.transpose(-2, -1), torch.eye(16, dtype=torch.float64).expand(3, 16, 16), atol=1e-9)
    q = bu.orth_quality(p[0], x[0])
    assert q["cosine"] > 1 - 1e-9 and q["rel_fro_err"] < 1e-9 and abs(q["sv_min"] - 1) < 1e-9
    assert bool((bu.batched_polar_cosine(p, x) > 1 - 1e-9).all())
    t = bu.measure(lambda: x @ x.transpose(-2, -1), warmup=1, iters=4, keep_raw=True)
    assert t["iters"] == 4 and len(t["raw_ms"]) == 4 and t["p25_ms"] <= t["median_ms"] <= t["p75_ms"]
    r = bu.measure_paired_speedup(lambda: x @ x.transpose(-2, -1), lambda: x + 1, warmup=1, iters=3)
    assert r["speedup_p25"] <= r["speedup_median"] <= r["speedup_p75"]


def test_result_io_and_tables(tmp_path):
    path = bu.save_results("demo", {"a": torch.tensor([1.0, 2.0]), "b": (1, 2)}, str(tmp_path))
    back = bu.load_results("demo", str(tmp_path))
    assert back["experiment"] == "demo" and back["data"] == {"a": [1.0, 2.0], "b": [1, 2]} and os.path.exists(path)
    txt = ps.text_table(("x", "y"), [(1, 0.5), (20, None)])
    assert txt.splitlines()[0].split() == ["x", "y"] and "-" in txt.splitlines()[2]
    out = ps.bar_chart(["a", "b"], {"s": [1.0, 2.0]}, "ms", "t", str(tmp_path), "bars", errors={"s": ([0.5, 1.5], [1.5, 2.5])})
    assert os.path.exists(os.path.join(tmp_path, "bars.txt")) and os.path.exists(out)
    ps.line_chart([1, 2], {"s": [1.0, 2.0]}, "x", "y", "t", str(tmp_path), "lines", bands={"s": ([0.9, 1.9], [1.1, 2.1])})
    ps.heatmap(["r0"], ["c0", "c1"], [[1.5, None]], "t", str(tmp_path), "heat", center=1.0)
    assert {"lines.txt", "heat.txt"} <= set(os.listdir(tmp_path))
    tex = ps.latex_table(("m", "v"), [("a", 1.0)], caption="c", label="l")
    assert r"\toprule" in tex and r"\caption{c}" in tex


def test_assoc_mem_engine_invariants():
    prob = am.sample_problem(64, 512, "power_law", 1.5, seed=0)
    assert abs(float(prob.p.sum()) - 1.0) < 1e-5 and bool((prob.p[:-1] >= prob.p[1:]).all())
    g_pop, meta = am.build_gradient(prob, "approx_population")
    assert meta["effective_support"] == 512 and g_pop.shape == (64, 64)
    g_mb, meta = am.build_gradient(prob, "true_minibatch", batch_size=640, seed=3)
    assert 0 < meta["effective_support"] < 512
    with pytest.raises(ValueError):
        am.build_gradient(prob, "true_minibatch")
    # tiling round trip, and a tile that covers the matrix is plain Muon
    tiled, info = am.tile_matrix(g_mb, (16, 32))
    assert torch.equal(am.untile_matrix(tiled, info), g_mb)
    assert torch.allclose(am.himuon_operator(g_mb, 64), am.himuon_operator(g_mb, None))
    # orthogonalised updates recover more than the raw gradient, larger tiles more than smaller ones
    counts = {}
    for label, opt, tile in (("sgd", "sgd", None), ("muon", "muon", None), ("t32", "himuon", 32), ("t16", "himuon", 16)):
        ok, margin = am.evaluate_recovery(prob, am.apply_one_step(g_mb, opt, 1.0, 5, tile or 64))
        counts[label] = int(ok.sum())
        assert bool(((margin > 0) == ok).all())
    assert counts["muon"] >= counts["t32"] >= counts["t16"] > counts["sgd"]
    # recovery does not depend on the step size
    a, _ = am.evaluate_recovery(prob, am.apply_one_step(g_mb, "muon", 1.0))
    b, _ = am.evaluate_recovery(prob, am.apply_one_step(g_mb, "muon", 0.01))
    assert torch.equal(a, b)
    # precision ladder: the gap to fp64 grows as the arithmetic gets coarser
    ref = am.himuon_operator(g_mb, 32, 5, "fp64_ref")
    gaps = [am.operator_gap_metrics(ref, am.himuon_operator(g_mb, 32, 5, p))["operator_relative_fro_gap"]
            for p in ("fp32", "bf16", "fp8e4m3_sim")]
    assert gaps[0] < 1e-4 < gaps[1] and gaps[0] < gaps[2]
    m = am.recovery_metrics(prob, am.apply_one_step(g_mb, "muon", 1.0), topk_values=(8, 32))
    assert m["recovered_count"] == counts["muon"] and 0 <= m["freq_top_8_recovered_fraction"] <= 1
    curve = am.topk_recovery_curve(prob, am.apply_one_step(g_mb, "muon", 1.0), max_k=16)
    assert curve["max_k"] == 16 and len(curve["topk_recovered_fraction"]) == 16
    with pytest.raises(MemoryError):
        am.assert_memory_budget(0.001, d=1024, num_items=100000)


EXPERIMENTS = [
    ("ns_convergence", ["--D", "128", "--max-k", "5", "--tiles", "32", "64", "--seeds", "1"]),
    ("capacity_scaling", ["--ds", "64", "--alphas", "1.5", "--num-items", "512", "--seeds", "0", "--tiles", "16", "32", "--no-jsonl"]),
    ("topk_recovery", ["--d", "64", "--num-items", "512", "--seeds", "0", "1", "--tiles", "16", "32"]),
    ("precision_recovery", ["--d", "64", "--num-items", "256", "--seeds", "0", "1", "--tiles", "16", "32"]),
    ("precision_descent", ["--dim", "64", "--steps", "5", "--tiles", "16", "32", "--batch", "32"]),
    ("tile_shape_quality", ["--model", "tiny-llama", "--shapes", "64x64", "16x64", "--steps", "12", "--batch", "2", "--seq", "32",
                            "--tail", "4", "--vocab", "64", "--warmup-steps", "2", "--decay-steps", "4"]),
    ("ns_kernel_microbench", ["--batches", "2", "--T", "32", "--warmup", "1", "--repeats", "2"]),
    ("ns5_rect_bench", ["--total-elements", "2048", "--dims", "16", "32", "--warmup", "1", "--repeats", "2"]),
    ("optimizer_step_microbench", ["--sizes", "64", "--K", "2", "--tile", "32", "--warmup", "1", "--repeats", "2"]),
    ("real_shapes_bench", ["--models", "tiny-qwen3", "--tile", "32", "--warmup", "1", "--repeats", "2", "--sweep-tiles", "32"]),
]


@pytest.mark.parametrize("name,argv", EXPERIMENTS, ids=[e[0] for e in EXPERIMENTS])
def test_experiment_runs_stores_and_replots(name, argv, tmp_path, capsys):
    import importlib

    mod = importlib.import_module(f"microbench.experiments.exp_{name}")
    dirs = ["--data-dir", str(tmp_path / "data"), "--out-dir", str(tmp_path / "plots")]
    data = mod.main(argv + dirs)
    stored = json.load(open(tmp_path / "data" / f"{name}.json"))
    assert stored["experiment"] == name and stored["data"].keys() == data.keys()
    assert any(f.endswith(".txt") for f in os.listdir(tmp_path / "plots"))
    capsys.readouterr()
    mod.main(["--plot-only"] + dirs)                       # re-plot from the stored JSON, nothing measured
    assert "saved" not in capsys.readouterr().out
    if name == "ns_convergence":
        cos = data["series"]["32"]["cos"]
        assert cos[-1] > 0.97 and cos[-1] > cos[0]
    if name == "ns_kernel_microbench":
        assert all(a["cosine_vs_fp32"] > 0.99 for r in data["rows"] for a in r["arms"].values())
    if name == "precision_descent":
        assert data["loss"][-1] < data["loss"][0]
        assert all(0 < g <= 1.5 for g in data["curves"]["full/fp32"]["gamma"])
    if name == "precision_recovery":
        assert os.path.exists(tmp_path / "plots" / "precision_recovery_table.tex")
    if name == "tile_shape_quality":
        assert all(r["full_matrix_buckets"] == 0 and r["losses"][-1] < r["losses"][0] for r in data["rows"])


def test_runner_registry_and_forwarded_flags(tmp_path):
    from microbench import plot as mb_plot
    from microbench import run as mb_run

    assert mb_run.TESTS["shapes"] == "real_shapes_bench" and mb_run._resolve("ns_convergence") == "ns_convergence"
    assert mb_run._resolve("precision_descent") == "precision_descent"
    with pytest.raises(SystemExit):
        mb_run._resolve("nope")
    dirs = ["--data-dir", str(tmp_path / "d"), "--out-dir", str(tmp_path / "p")]
    mb_run.main(["--test", "ns_convergence", "--sizes", "64", "--no-plot"] + dirs)
    stored = json.load(open(tmp_path / "d" / "ns_convergence.json"))
    assert stored["data"]["D"] == 64 and not os.path.exists(tmp_path / "p")
    mb_plot.main(dirs)
    assert "ns_convergence.txt" in os.listdir(tmp_path / "p")
