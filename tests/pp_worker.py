"""Worker of the pipeline-parallel GPU test: run with ``torch.distributed.run --nproc-per-node 2``.

Two stages, one GPU each, of the same tiny model.  Every stage makes the same engine calls; the
first stage plans, each stage saves and restores the KV of its own layers in a store file of
its own, the residual stream travels over NCCL point-to-point, and the last stage samples.
Stage 0 then runs the whole model on its GPU alone and the tokens must agree: cold (chunks
computed), warm (chunks restored from each stage's store), and while decoding.
Prints ``PP_OK`` when everything agrees.
"""

import asyncio
import os
import random
import sys
import tempfile
import threading

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from daser_b200.config import DaserConfig  # noqa: E402
from daser_b200.engine.rag_gpu import GpuRagEngine  # noqa: E402
from daser_b200.models.llama import PRESETS  # noqa: E402
from daser_b200.parallel.pp import StageLink, stage_geometry  # noqa: E402
from daser_b200.server.__main__ import ControlPlane  # noqa: E402


def _plane(dcfg):
    plane = ControlPlane(dcfg)
    loop = asyncio.new_event_loop()
    ready = threading.Event()

    def serve():
        asyncio.set_event_loop(loop)
        loop.run_until_complete(plane.start())
        ready.set()
        loop.run_forever()

    threading.Thread(target=serve, daemon=True).start()
    ready.wait(20)
    return plane, loop


def main() -> None:
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stages = dist.get_world_size()
    cfg = PRESETS["tiny-gqa"]
    link = StageLink()
    tmp = link.from_stage(tempfile.mkdtemp(prefix="daser_pp_") if rank == 0 else None, 0)
    geo = stage_geometry(cfg, stages, 2, "fp8b16")  # slots hold the widest stage's layers
    dcfg = DaserConfig(store_path=f"{tmp}/daser.store", index_path="", total_slots=128, slot_size=geo.slot_size,
                       ipc_socket_path=f"{tmp}/d.sock")
    plane = loop = None
    if rank == 0:
        plane, loop = _plane(dcfg)
    dist.barrier(device_ids=[local])
    eng = GpuRagEngine(cfg, dcfg.ipc_socket_path, dcfg.store_path, num_blocks=128, max_tokens=128, max_seqs=8,
                       hbm_slots=32, staging_slots=64, seed=5, pp_link=link)
    rng = random.Random(0)
    chunks = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (64, 96)]
    query = [rng.randrange(cfg.vocab_size) for _ in range(12)]
    checks = {"layers": eng.runner.layers == range(rank * cfg.num_layers // stages, (rank + 1) * cfg.num_layers // stages)}
    cold = eng.generate([chunks[1], chunks[0]], query, max_new_tokens=4)  # nothing stored: all computed
    for c in chunks:
        eng.store_chunk(c)  # every stage writes its layers, the chunk appears when both have committed
    for tier in (eng.hbm, eng.host):
        if tier is not None:
            tier.clear()
    filed = eng.generate([chunks[1], chunks[0]], query, max_new_tokens=4)  # from the stages' store files
    warm = eng.generate([chunks[1], chunks[0]], query, max_new_tokens=4)  # from the stages' HBM tiers
    eng.runner.check_status()
    checks["restored"] = (cold.restored_chunks, filed.restored_chunks, warm.restored_chunks) == (0, 2, 2)
    checks["file_equals_tier"] = filed.generated == warm.generated and len(cold.generated) == 4
    everyone = link.gather_object((cold.generated, filed.generated))
    checks["same_on_every_stage"] = all(e == everyone[0] for e in everyone)
    ok = all(checks.values())
    if not ok:
        print(f"stage {rank}: {checks} restored={cold.restored_chunks, filed.restored_chunks, warm.restored_chunks} "
              f"filed={filed.generated} warm={warm.generated}", flush=True)
    eng.close()
    if rank == 0:
        # the whole model on one GPU, same seed: same weights tensor by tensor
        dcfg1 = DaserConfig(store_path=f"{tmp}/single.store", index_path="", total_slots=128,
                            slot_size=cfg.num_layers * 2 * 16 * cfg.num_kv_heads * cfg.head_dim * 5 // 4,
                            ipc_socket_path=f"{tmp}/d1.sock")
        plane1, loop1 = _plane(dcfg1)
        single = GpuRagEngine(cfg, dcfg1.ipc_socket_path, dcfg1.store_path, num_blocks=128, max_tokens=128,
                              max_seqs=8, hbm_slots=32, staging_slots=64, seed=5)
        cold1 = single.generate([chunks[1], chunks[0]], query, max_new_tokens=4)
        for c in chunks:
            single.store_chunk(c)
        warm1 = single.generate([chunks[1], chunks[0]], query, max_new_tokens=4)
        single.close()
        print(f"pipeline cold={cold.generated} warm={warm.generated}; single cold={cold1.generated} "
              f"warm={warm1.generated}", flush=True)
        ok = ok and cold.generated == cold1.generated and warm.generated == warm1.generated
        for p, l in ((plane, loop), (plane1, loop1)):
            asyncio.run_coroutine_threadsafe(p.stop(save=False), l).result(10)
            l.call_soon_threadsafe(l.stop)
    flags = link.gather_object(bool(ok))
    if rank == 0:
        print("PP_OK" if all(flags) else f"PP_FAIL {flags}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
