import json

from daser_b200.utils import trace


def test_spans_are_written_as_chrome_trace(tmp_path):
    path = str(tmp_path / "t.json")
    trace.clear()
    trace.enable(path)
    try:
        with trace.span("outer", "test", n=3):
            with trace.span("inner"):
                pass
        trace.instant("mark", k=1)
        assert trace.dump() == path
    finally:
        trace.disable()
        trace.clear()
    ev = json.load(open(path))["traceEvents"]
    names = [e["name"] for e in ev]
    assert names == ["inner", "outer", "mark"]
    outer = ev[1]
    assert outer["ph"] == "X" and outer["dur"] >= ev[0]["dur"] and outer["args"] == {"n": 3}


def test_disabled_tracing_records_nothing():
    trace.clear()
    with trace.span("x"):
        pass
    assert trace.dump() is None


def test_connector_hooks_are_traced(tmp_path):
    import random

    from conftest import LiveControlPlane
    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.kv.layout import KVGeometry
    from daser_b200.models.llama import PRESETS

    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, 16, 4, "raw")
    lp = LiveControlPlane(tmp_path, total_slots=32, slot_size=geo.slot_size).start()
    eng = CpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=32)
    trace.clear()
    trace.enable(str(tmp_path / "c.json"))
    try:
        chunk = [random.Random(0).randrange(32000) for _ in range(32)]
        eng.store_chunk(chunk)
        eng.run_request([1] * 16, [chunk], [2, 3])
        trace.dump()
    finally:
        trace.disable()
        eng.close()
        lp.stop()
    names = {e["name"] for e in json.load(open(tmp_path / "c.json"))["traceEvents"]}
    assert {"wait_for_save", "start_load_kv", "rpc.lookup_chunks", "io.reads_submitted"} <= names
    trace.clear()
