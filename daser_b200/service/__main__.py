"""``python -m daser_b200.service`` — REST service with the control plane embedded.

Capability parity: ``daser/service/__main__.py:26-213`` — flags ``--host`` (0.0.0.0),
``--port`` (8080), ``--vllm-base-url``, ``--model``, ``--tokenizer``, ``--socket-path``,
``--store-path``, ``--index-path``, ``--total-slots`` (1024), ``--slot-size`` (0 = derive),
``--block-tokens``, ``--chunk-blocks``, the model-geometry flags and ``--model-id``; the
control plane and uvicorn share one event loop, and a snapshot is written on shutdown.

Added: ``--engine native`` serves from the in-process engine (``--native-model`` names a
preset; ``cpu`` or ``cuda`` device) instead of a remote vLLM, in which case
``--vllm-base-url`` and ``--model`` are optional.
"""

from __future__ import annotations

import argparse
import asyncio
import os
import signal
from typing import Optional, Sequence

from daser_b200.config import DaserConfig
from daser_b200.logging import init_logger
from daser_b200.server.__main__ import ControlPlane
from daser_b200.service.http_api import ServiceConfig, build_service_app, load_tokenizer

logger = init_logger(__name__)


def _parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="daser_b200.service", description=__doc__)
    p.add_argument("--host", default="0.0.0.0")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--engine", choices=("vllm", "native"), default="vllm")
    p.add_argument("--vllm-base-url", default=None)
    p.add_argument("--model", default=None)
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--socket-path", default="/tmp/daser.sock")
    p.add_argument("--store-path", default="/mnt/xfs/daser.store")
    p.add_argument("--index-path", default="/mnt/xfs/daser.index")
    p.add_argument("--total-slots", type=int, default=1024)
    p.add_argument("--slot-size", type=int, default=0)
    p.add_argument("--block-tokens", type=int, default=16)
    p.add_argument("--chunk-blocks", type=int, default=16)
    p.add_argument("--num-kv-heads", type=int, default=0)
    p.add_argument("--head-dim", type=int, default=0)
    p.add_argument("--num-layers", type=int, default=0)
    p.add_argument("--dtype-bytes", type=int, default=2)
    p.add_argument("--model-id", default="default")
    p.add_argument("--native-model", default="toy")
    p.add_argument("--native-device", choices=("cpu", "cuda"), default="cpu")
    p.add_argument("--native-max-in-flight", type=int, default=0,
                   help="with --native-batching: answer 429 above this many unfinished requests (0 = no limit)")
    p.add_argument("--native-checkpoint", default=None,
                   help="directory of a Hugging Face checkpoint (config.json + *.safetensors; Llama-3 and Qwen3 "
                        "families): architecture and weights of the native engine instead of --native-model "
                        "with random weights")
    p.add_argument("--native-compose-after", type=int, default=0,
                   help="store an ordered chunk combination whole after this many sightings and restore it as "
                        "one exact chunk later (0 = off)")
    p.add_argument("--native-repair-tokens", type=int, default=0,
                   help="recompute the first N tokens of every chunk restored behind other context (0 = off)")
    p.add_argument("--native-batching", action="store_true",
                   help="one thread keeps the native engine stepping and concurrent requests share its steps "
                        "(continuous batching); without it requests are served one after the other")
    p.add_argument("--snapshot-interval", type=float, default=0.0)
    p.add_argument("--no-fast-lookup", action="store_true",
                   help="do not start the native thread that answers lookups by key on <socket>.fast")
    args = p.parse_args(argv)
    if args.no_fast_lookup:
        os.environ["DASER_FAST_LOOKUP"] = "0"
    if args.engine == "vllm" and (not args.vllm_base_url or not args.model):
        p.error("--vllm-base-url and --model are required with --engine vllm")
    return args


def _build_daser_config(args: argparse.Namespace) -> DaserConfig:
    return DaserConfig(
        store_path=args.store_path, index_path=args.index_path, total_slots=args.total_slots,
        slot_size=args.slot_size, ipc_socket_path=args.socket_path, num_kv_heads=args.num_kv_heads,
        head_dim=args.head_dim, num_layers=args.num_layers, block_tokens=args.block_tokens,
        dtype_bytes=args.dtype_bytes, model_id=args.model_id,
        snapshot_interval_s=getattr(args, "snapshot_interval", 0.0),
    )


def _world() -> tuple[int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


_TP_CTX = None


def _tp_context(mcfg):
    """The tensor-parallel context when the service was started under torchrun with several
    ranks (one per GPU); None for a single process."""
    global _TP_CTX
    rank, world = _world()
    if world <= 1:
        return None
    if _TP_CTX is None:
        import torch
        import torch.distributed as dist

        from daser_b200.parallel.tp import TPContext

        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        torch.cuda.set_device(local)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        _TP_CTX = TPContext(mcfg, dist.group.WORLD, max_tokens=256)
    return _TP_CTX


def _model_config(args: argparse.Namespace):
    """The native engine's architecture: a preset name, or the ``config.json`` of ``--native-checkpoint``."""
    from daser_b200.models.llama import PRESETS

    if getattr(args, "native_checkpoint", None):
        import json

        from daser_b200.models.hf import config_from_hf

        with open(os.path.join(args.native_checkpoint, "config.json")) as f:
            return config_from_hf(json.load(f), name=os.path.basename(os.path.normpath(args.native_checkpoint)),
                                  block_tokens=args.block_tokens)
    return PRESETS[args.native_model]


def _model_weights(args: argparse.Namespace, device, dtype, tp: int = 1, rank: int = 0):
    """This rank's shard of the checkpoint, or None (the engine then draws random weights)."""
    if not getattr(args, "native_checkpoint", None):
        return None
    from daser_b200.models.hf import load_checkpoint

    return load_checkpoint(args.native_checkpoint, tp=tp, rank=rank, dtype=dtype, device=device,
                           block_tokens=args.block_tokens)


def _engine_options(args: argparse.Namespace) -> dict:
    return {"compose_after": int(getattr(args, "native_compose_after", 0) or 0),
            "repair_tokens": int(getattr(args, "native_repair_tokens", 0) or 0)}


def _eos_ids(args: argparse.Namespace) -> tuple:
    """End-of-sequence ids of a checkpoint (``generation_config.json``, else ``config.json``); none for
    the presets with random weights, whose generations run to ``max_tokens``."""
    if not getattr(args, "native_checkpoint", None):
        return ()
    import json

    ids: list[int] = []
    for name in ("generation_config.json", "config.json"):
        path = os.path.join(args.native_checkpoint, name)
        if os.path.exists(path):
            with open(path) as f:
                eos = json.load(f).get("eos_token_id")
            if eos is not None:
                ids = [int(t) for t in (eos if isinstance(eos, list) else [eos])]
                break
    return tuple(ids)


def _run_follower(args: argparse.Namespace) -> None:
    """Ranks above 0: build the same engine shard and replay the leader's calls until told to stop."""
    import torch

    from daser_b200.engine.rag_gpu import GpuRagEngine
    from daser_b200.service.tp_serving import follower_loop

    cfg = _build_daser_config(args)
    mcfg = _model_config(args)
    tp_ctx = _tp_context(mcfg)
    tp_ctx.barrier()  # the leader's control plane is up
    engine = GpuRagEngine(mcfg, cfg.ipc_socket_path, cfg.store_path, model_id=cfg.model_id,
                          hbm_slots=min(cfg.total_slots, 4096), tp_ctx=tp_ctx,
                          weights=_model_weights(args, "cuda", torch.bfloat16, tp_ctx.tp, tp_ctx.rank),
                          **_engine_options(args))
    steps = follower_loop(engine, tp_ctx.await_announcement)  # idle between requests: no time limit, peers watched
    logger.info("[SERVICE] follower rank %d leaves after %d engine calls", tp_ctx.rank, steps)


def _native_engine(args: argparse.Namespace, cfg: DaserConfig, tokenizer):
    import torch

    from daser_b200.service.vllm_client import NativeEngineClient

    mcfg = _model_config(args)
    if args.native_device == "cuda":
        from daser_b200.engine.rag_gpu import GpuRagEngine

        tp_ctx = _tp_context(mcfg)
        shard = (tp_ctx.tp, tp_ctx.rank) if tp_ctx is not None else (1, 0)
        engine = GpuRagEngine(mcfg, cfg.ipc_socket_path, cfg.store_path, model_id=cfg.model_id,
                              hbm_slots=min(cfg.total_slots, 4096), tp_ctx=tp_ctx,
                              weights=_model_weights(args, "cuda", torch.bfloat16, *shard), **_engine_options(args))
        if tp_ctx is not None:
            from daser_b200.service.tp_serving import TPLeaderEngine

            # rank 0 leads: every engine call is announced to the followers first
            engine = TPLeaderEngine(engine, tp_ctx.broadcast_object)
    else:
        from daser_b200.engine.rag_cpu import CpuRagEngine

        engine = CpuRagEngine(mcfg, cfg.ipc_socket_path, cfg.store_path, model_id=cfg.model_id,
                              weights=_model_weights(args, "cpu", torch.float32), **_engine_options(args))
    return NativeEngineClient(engine, tokenizer.decode, model=args.native_model,
                              batching=bool(getattr(args, "native_batching", False)), eos_token_ids=_eos_ids(args),
                              max_in_flight=int(getattr(args, "native_max_in_flight", 0) or 0)), engine


async def _run(args: argparse.Namespace) -> None:
    import uvicorn

    cfg = _build_daser_config(args)
    tokenizer = load_tokenizer(args.tokenizer)
    engine_client = engine = None
    if args.engine == "native":
        m = _model_config(args)
        if cfg.slot_size == 0 and cfg.num_layers == 0:
            cfg.num_layers, cfg.num_kv_heads, cfg.head_dim = m.num_layers, m.num_kv_heads, m.head_dim
            cfg.dtype_bytes = 4 if args.native_device == "cpu" else 2
            cfg.codec = "raw" if args.native_device == "cpu" else "fp8b16"
    plane = ControlPlane(cfg)
    await plane.start()
    if args.engine == "native":
        if args.native_device == "cuda" and _world()[1] > 1:
            _tp_context(_model_config(args)).barrier()  # followers may connect to the control plane now
        # built off the loop: the engine's connector talks to the control plane, which this loop serves
        engine_client, engine = await asyncio.get_running_loop().run_in_executor(
            None, _native_engine, args, cfg, tokenizer)
    app = build_service_app(
        ServiceConfig(vllm_base_url=args.vllm_base_url or "", model=args.model or args.native_model,
                      tokenizer=args.tokenizer, socket_path=args.socket_path, block_tokens=args.block_tokens,
                      chunk_blocks=args.chunk_blocks),
        engine_client=engine_client, tokenizer=tokenizer,
    )
    if args.engine == "native":
        # the in-process engine also answers vLLM's completions API (token-id prompts), with the
        # stored chunks of a prompt found by a scan: a client written for vLLM can point here
        from daser_b200.service.openai_api import mount_openai_routes

        mount_openai_routes(app, engine_client, tokenizer, args.socket_path, args.native_model, cfg.model_id,
                            args.block_tokens)
    server = uvicorn.Server(uvicorn.Config(app, host=args.host, port=args.port, loop="none", log_level="info"))
    stop = asyncio.Event()
    loop = asyncio.get_running_loop()
    for sig in (signal.SIGTERM, signal.SIGINT):
        loop.add_signal_handler(sig, stop.set)
    http_task = asyncio.create_task(server.serve())
    stop_task = asyncio.create_task(stop.wait())
    await asyncio.wait({http_task, stop_task}, return_when=asyncio.FIRST_COMPLETED)
    server.should_exit = True
    await asyncio.gather(http_task, return_exceptions=True)
    stop_task.cancel()
    if engine_client is not None and engine is not None:
        await engine_client.close()  # drains the engine loop, if there is one, before the engine goes
    if engine is not None:
        engine.close()
    await plane.stop(save=True)


def main(argv: Optional[Sequence[str]] = None) -> None:
    args = _parse_args(argv)
    rank, world = _world()
    if world > 1 and rank > 0:
        if args.engine != "native" or args.native_device != "cuda":
            return  # nothing to do on extra ranks of a single-process configuration
        _run_follower(args)
        return
    asyncio.run(_run(args))


if __name__ == "__main__":
    main()
