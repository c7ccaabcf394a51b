"""This package's connector under a real, stock ``vllm.LLM`` on one GPU.

Cold engine: every prompt misses, is prefilled, and its KV is stored through the fused save
kernel.  A second, new engine process then serves the same prompts: they hit, the KV comes back
from the store file through the fused restore kernel, and greedy decoding must continue exactly
as it did in the cold run.  Run once per KV layout vLLM offers on the box (FlashAttention's
``(2, blocks, ...)`` and FlashInfer's ``(blocks, 2, ...)``), with the raw and the fp8 codec.
"""

import json
import os
import subprocess
import sys

import pytest

from conftest import LiveControlPlane

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L, H, D, B = 2, 2, 128, 16  # the tiny-gqa model: layers, KV heads, head dim, block tokens


def _phase(tmp_path, lp, backend, codec):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import vllm_common as vc

    env = vc.clean_env([ROOT, os.path.join(ROOT, "baseline")])
    env["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
    cmd = [sys.executable, os.path.join(ROOT, "tests", "vllm_worker.py"), "--socket", lp.socket_path, "--store",
           lp.cfg.store_path, "--model-dir", str(tmp_path / "model"), "--backend", backend, "--codec", codec]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    lines = [l for l in proc.stdout.splitlines() if l.startswith("VLLM_RESULT ")]
    assert proc.returncode == 0 and lines, (proc.stdout + proc.stderr)[-4000:]
    return json.loads(lines[-1][len("VLLM_RESULT "):])


@pytest.mark.parametrize("backend,codec", [("FLASH_ATTN", "raw"), ("FLASHINFER", "fp8b16")])
def test_cold_engine_stores_and_a_new_engine_restores(tmp_path, backend, codec):
    pytest.importorskip("vllm")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import vllm_common as vc

    vc.write_hf_config("tiny-gqa", str(tmp_path / "model"), max_positions=8192)
    per_elem = 2 if codec == "raw" else 1.25
    slot = int(L * 2 * B * H * D * per_elem)
    lp = LiveControlPlane(tmp_path, total_slots=256, slot_size=slot).start()
    try:
        cold = _phase(tmp_path, lp, backend, codec)
        assert cold["bytes_stored"] > 0 and cold["bytes_loaded"] == 0 and cold["prefix_hits"] == 0
        warm = _phase(tmp_path, lp, backend, codec)
        assert warm["prefix_hits"] == 3 and warm["load_errors"] == 0
        # 150, 83 and 260 prompt tokens: 9 + 5 + 16 whole blocks come back from the store
        assert warm["bytes_loaded"] == (9 + 5 + 16) * slot
        if codec == "raw":
            assert warm["tokens"] == cold["tokens"]  # bit-identical KV: greedy decoding repeats exactly
        else:
            # fp8 KV is not the KV the cold run attended to, and a random-init model's logits are
            # nearly flat, so tokens may part ways; the restore's numerics are pinned by the kernel
            # tests.  Here: the engine decoded to the end on restored fp8 KV.
            assert [len(w) for w in warm["tokens"]] == [len(c) for c in cold["tokens"]]
    finally:
        lp.stop()
