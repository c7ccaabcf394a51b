"""Child process of ``tests/test_gpu_vllm_real.py``: one stock ``vllm.LLM`` with this package's
connector, one pass over a few prompts, results as one JSON line.

The parent keeps the control plane and the store file alive across two such children: the first
(cold) computes and stores, the second (warm) is a new engine that restores what the first one
stored.  This is the shape of the reference's only integration test
(``tests/integration/test_vllm_e2e.py:127-196`` there: cold generate -> new engine -> warm
generate, outputs identical).  The engine core runs inside this process so that the connector's
counters can be read afterwards.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--socket", required=True)
    ap.add_argument("--store", required=True)
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--backend", default="FLASH_ATTN")
    ap.add_argument("--codec", default="raw")
    ap.add_argument("--tokens", type=int, default=16)
    args = ap.parse_args()
    os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"

    import random

    import vllm_common as vc
    from vllm import SamplingParams
    from vllm.inputs import TokensPrompt

    from daser_b200 import metrics

    rng = random.Random(11)
    prompts = [[rng.randrange(3, 1000) for _ in range(n)] for n in (150, 83, 260)]
    ktc = {
        "kv_connector": "DaserConnector",
        "kv_connector_module_path": "daser_b200.connector.daser_connector",
        "kv_role": "kv_both",
        "kv_connector_extra_config": {"socket_path": args.socket, "store_path": args.store, "block_tokens": 16,
                                      "model_id": "tiny-gqa", "codec": args.codec, "hbm_slots": 64},
    }
    llm = vc.build_llm(args.model_dir, 1, ktc, max_model_len=1024, gpu_memory_utilization=0.3,
                       attention_backend=args.backend, enforce_eager=True)
    params = SamplingParams(temperature=0.0, max_tokens=args.tokens, detokenize=False)
    t0 = time.perf_counter()
    outs = llm.generate([TokensPrompt(prompt_token_ids=p) for p in prompts], params, use_tqdm=False)
    dt = time.perf_counter() - t0
    snap = metrics.snapshot()
    result = {
        "tokens": [list(o.outputs[0].token_ids) for o in outs],
        "seconds": round(dt, 3),
        "bytes_loaded": snap.get("connector.bytes_loaded", 0),
        "bytes_stored": snap.get("connector.bytes_stored", 0),
        "prefix_hits": snap.get("connector.prefix_hits", 0),
        "load_errors": snap.get("connector.load_errors", 0),
    }
    print("VLLM_RESULT " + json.dumps(result), flush=True)
    vc.destroy_llm(llm)


if __name__ == "__main__":
    main()
