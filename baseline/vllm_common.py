"""Helpers for driving the stock ``vllm.LLM`` offline with a random-init model.

Used by the reference arm of the headline benchmark (``baseline/reference_arm.py``) and by the
GPU test that runs this framework's connector under a real vLLM.  Imports neither
implementation.
"""

from __future__ import annotations

import json
import os
import subprocess
import tempfile
import time
from typing import Any, Optional

from traffic import MODEL_SHAPES

TORCHRUN_VARS = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE",
                 "ROLE_RANK", "ROLE_WORLD_SIZE", "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID",
                 "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_USE_AGENT_STORE",
                 "TORCH_NCCL_ASYNC_ERROR_HANDLING", "TORCHELASTIC_ERROR_FILE", "OMP_NUM_THREADS")


def clean_env(extra_pythonpath: list[str]) -> dict[str, str]:
    """The environment for a vLLM process that manages its own workers: no launcher variables,
    no network look-ups, the given directories importable in every child it spawns."""
    env = {k: v for k, v in os.environ.items() if k not in TORCHRUN_VARS}
    old = env.get("PYTHONPATH", "")
    env["PYTHONPATH"] = os.pathsep.join(extra_pythonpath + ([old] if old else []))
    env.update(HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1", VLLM_NO_USAGE_STATS="1", DO_NOT_TRACK="1",
               VLLM_WORKER_MULTIPROC_METHOD="spawn", PYTHONHASHSEED="0", TOKENIZERS_PARALLELISM="false")
    env.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    # the reference logs every block id of every request at INFO (its own variable: daser/logging.py:31)
    env.setdefault("DASER_LOG_LEVEL", "WARNING")
    return env


def write_hf_config(model: str, directory: str, max_positions: int = 131072) -> str:
    """A Hugging Face ``config.json`` of the named architecture (weights are random: ``load_format="dummy"``)."""
    s = MODEL_SHAPES[model]
    cfg: dict[str, Any] = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "hidden_size": s["hidden_size"], "intermediate_size": s["intermediate_size"],
        "num_hidden_layers": s["num_hidden_layers"], "num_attention_heads": s["num_attention_heads"],
        "num_key_value_heads": s["num_key_value_heads"], "head_dim": s["head_dim"], "vocab_size": s["vocab_size"],
        "rms_norm_eps": s["rms_norm_eps"], "rope_theta": s["rope_theta"], "max_position_embeddings": max_positions,
        "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_bias": False, "mlp_bias": False,
        "bos_token_id": 1, "eos_token_id": 2, "initializer_range": 0.02, "use_cache": True,
    }
    if s.get("llama3_scaling"):
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192}
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(cfg, f)
    return directory


def slot_size_bf16(model: str, block_tokens: int = 16, tp: int = 1) -> int:
    """Bytes of one block's KV over all layers as one rank of a ``tp``-way engine holds it."""
    s = MODEL_SHAPES[model]
    heads = max(1, s["num_key_value_heads"] // tp)
    return heads * s["head_dim"] * 2 * s["num_hidden_layers"] * block_tokens * 2


def build_llm(model_dir: str, tp: int, kv_transfer_config: Optional[dict], max_model_len: int,
              gpu_memory_utilization: float = 0.9, attention_backend: Optional[str] = "FLASH_ATTN",
              enforce_eager: bool = False, max_num_seqs: int = 8, block_size: int = 16):
    from vllm import LLM

    kwargs: dict[str, Any] = dict(
        model=model_dir, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", seed=0,
        tensor_parallel_size=tp, gpu_memory_utilization=gpu_memory_utilization, max_model_len=max_model_len,
        max_num_batched_tokens=max_model_len, max_num_seqs=max_num_seqs, enable_prefix_caching=False,
        block_size=block_size, enforce_eager=enforce_eager, disable_custom_all_reduce=True,
        disable_log_stats=True, generation_config="vllm",
    )
    if tp > 1:
        kwargs["distributed_executor_backend"] = "mp"
    if attention_backend:
        kwargs["attention_backend"] = attention_backend
    if kv_transfer_config is not None:
        kwargs["kv_transfer_config"] = kv_transfer_config
        kwargs["disable_hybrid_kv_cache_manager"] = True
    return LLM(**kwargs)


def destroy_llm(llm) -> None:
    try:
        llm.llm_engine.engine_core.shutdown()
    except Exception:  # noqa: BLE001
        pass


def first_token_ms(llm, prompt_token_ids: list[int]) -> tuple[float, list[int]]:
    """Wall-clock time of one ``generate`` call that stops after the first token, and that token."""
    from vllm import SamplingParams
    from vllm.inputs import TokensPrompt

    params = SamplingParams(temperature=0.0, max_tokens=1, detokenize=False)
    t0 = time.perf_counter()
    out = llm.generate([TokensPrompt(prompt_token_ids=prompt_token_ids)], params, use_tqdm=False)
    dt = (time.perf_counter() - t0) * 1e3
    return dt, list(out[0].outputs[0].token_ids)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = os.path.join(tempfile.gettempdir(), f"daser_clocks_{os.getpid()}.csv")

    def start(self) -> None:
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}
