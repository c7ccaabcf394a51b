"""The parts of ``bench.py`` that need no GPU: traffic generation, the clock sampler's parsing,
and the reference arm's one-line answer."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_traffic_is_deterministic_block_aligned_and_skewed():
    import bench
    from daser_b200.models.llama import PRESETS

    cfg = PRESETS["llama3-70b"]
    prefix, pool, reqs = bench.make_traffic(cfg.vocab_size, cfg.block_tokens, 64, 8, 30)
    prefix2, pool2, reqs2 = bench.make_traffic(cfg.vocab_size, cfg.block_tokens, 64, 8, 30)
    assert (prefix, pool, reqs) == (prefix2, pool2, reqs2)
    bt = cfg.block_tokens
    assert len(prefix) == 64 and all(len(c) % bt == 0 and 64 <= len(c) <= 1024 for c in pool)
    for chunks, query, picked in reqs:
        assert chunks[0] is prefix and len(chunks) == 9 and len(query) == 64
        assert all(0 < t < cfg.vocab_size for t in query)
        assert [pool[i] for i in picked] == chunks[1:]
    # Zipf 1.1 over the pool: the few most popular chunks take a large share of the picks
    picks = [id(c) for chunks, _, _ in reqs for c in chunks[1:]]
    top = sorted((picks.count(id(c)) for c in pool), reverse=True)
    assert sum(top[:8]) > 0.4 * len(picks)
    ctx = [sum(map(len, chunks)) + len(q) for chunks, q, _ in reqs]
    assert 1500 < sum(ctx) / len(ctx) < 6000


def test_clock_sampler_parses_nvidia_smi_lines(tmp_path, monkeypatch):
    import bench

    s = bench.ClockSampler(0)
    s.path = str(tmp_path / "clocks.csv")
    with open(s.path, "w") as f:
        f.write("0, 1965, 1965, 420.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1710, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1850, 1965, 800.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n")
        f.write("garbage line\n")

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    s.proc, s.out = Done(), open(os.devnull, "w")
    got = s.stop()
    assert got == {"sm_mhz": 1850.0, "sm_max_mhz": 1965.0, "samples": 3, "reasons": ["sw_power_cap"]}
    assert bench.ClockSampler(0).stop()["reasons"] == ["nvidia-smi unavailable"]  # never started


def test_reference_arm_prints_one_json_line_and_exits_zero():
    for env in ({}, {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus",
                               env.get("WORLD_SIZE", "1"), "--steps", "2", "--warmup", "1"],
                              capture_output=True, text=True, timeout=120, env=dict(os.environ, **env))
        assert proc.returncode == 0, proc.stderr[-2000:]
        lines = [l for l in proc.stdout.splitlines() if l.strip()]
        if env.get("RANK") == "1":
            assert lines == []  # only rank 0 speaks
            continue
        assert len(lines) == 1
        out = json.loads(lines[0])
        assert out["impl"] == "reference" and ("unavailable" in out or "value" in out)
