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
