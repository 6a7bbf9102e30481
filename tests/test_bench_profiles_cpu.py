"""bench.py's `roofline.traffic` comes from the ncu summaries under profiles/, parsed at run time:
every entry of its table must resolve to a file that exists and to kernels found in it, so a stale
or renamed summary fails here rather than silently turning the figure into null."""
import bench


def test_every_traffic_entry_resolves_to_a_committed_summary():
    for (op, storage), (file, fragments, rows) in bench.PROFILE_TRAFFIC.items():
        path = bench.ROOT / "profiles" / file
        assert path.exists(), f"{op}/{storage}: {file} is missing"
        kernels = bench.parse_profile(path)
        for fragment in fragments:
            hits = [m for name, m in kernels if fragment in name]
            assert hits, f"{op}/{storage}: no kernel named *{fragment}* in {file}"
            assert hits[0]["dram read"] >= 0 and hits[0]["dram write"] >= 0 and hits[0]["duration"] > 0
        full = bench.ncu_traffic(op, storage, rows)
        assert full is not None and full > 0
        assert bench.ncu_traffic(op, storage, rows // 2) == full // 2 or abs(bench.ncu_traffic(op, storage, rows // 2) - full / 2) <= 1


def test_traffic_follows_the_file(tmp_path, monkeypatch):
    """Changing a number in a summary changes the figure bench.py reports."""
    file, fragments, rows = bench.PROFILE_TRAFFIC[("ln2_bwd", "bf16")]
    before = bench.ncu_traffic("ln2_bwd", "bf16", rows)
    text = (bench.ROOT / "profiles" / file).read_text()
    kernels = bench.parse_profile(bench.ROOT / "profiles" / file)
    read_mb = [m for name, m in kernels if fragments[0] in name][0]["dram read"] / 1e6
    (tmp_path / "profiles").mkdir()
    (tmp_path / "profiles" / file).write_text(text.replace(f"{read_mb:.6f} Mbyte", f"{read_mb + 100:.6f} Mbyte", 1))
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    after = bench.ncu_traffic("ln2_bwd", "bf16", rows)
    assert after == before + 100_000_000


def test_ops_without_a_capture_report_none():
    assert bench.ncu_traffic("allreduce", "bf16", 1024) is None
    assert bench.ncu_traffic("ln1_fwd", "fp32", 1024) is None


def test_table_of_a_recorded_line(tmp_path, capsys):
    """`python bench.py --table FILE` renders the chain ops and the kernel sweep of a recorded line."""
    import json
    line = {
        "n_gpus": 1, "dtype": "bf16", "ms_per_step": 1.5, "value": 2.0e7, "value_min": 1.9e7, "value_max": 2.1e7,
        "e2e": {"ms_per_step": 1.6, "value": 1.95e7}, "chain_gbs": 6000.0, "clocks": {"sm_mhz": 1965.0},
        "roofline": {"peak": 6556.8},
        "chain_ops": [{"op": "sort_tokens", "ms": 0.05, "bytes": 0, "gbs": None, "frac": None, "ncu_traffic": None},
                      {"op": "ln1_fwd", "ms": 0.17, "bytes": 1000, "gbs": 6100.0, "frac": 0.93, "ncu_traffic": 900}],
        "kernels_fp32": [{"kernel": "ln_bwd", "config": "65536x1024 fp32", "ms": 0.128, "gbs": 6300.0,
                          "frac_measured": 0.96, "ref_ms": 7.1, "speedup_vs_ref": 55.5, "max_rel_err_vs_ref": 1.5e-5,
                          "err_vs_fp64": {"dgamma": 9e-7}, "ref_err_vs_fp64": {"dgamma": 1.5e-5}},
                         {"kernel": "embed_sort_tokens", "config": "T32768", "ms": 0.05, "gbs": None}],
    }
    path = tmp_path / "line.json"
    path.write_text("noise\n" + json.dumps(line) + "\n")
    bench.print_table(path)
    out = capsys.readouterr().out
    assert "| ln1_fwd | 0.1700 | 6100 | 0.930 | 0.90 |" in out
    assert "| sort_tokens | 0.0500 | — | — | — |" in out
    assert "| ln_bwd | 65536x1024 fp32 | 0.1280 | 6300 | 0.960 | 7.1000 | 55.50x | 1.5e-05 | 9e-07 / 1.5e-05 |" in out
    assert "| embed_sort_tokens | T32768 | 0.0500 | — | — | — | — | — | — |" in out
