"""CPU ranks for the multi-process tests (``gloo`` backend, no GPU).

Scenarios, chosen by ``argv[1]``; RANK / WORLD_SIZE / MASTER_PORT come from the environment:

``parts``   two tensor-parallel workers in the per-rank-file arrangement used under vLLM: rank 0
            also runs the control plane and the scheduler half and broadcasts each step's plan;
            every rank stores its head slice into its own file and commits its part.  A chunk
            must be visible only after both parts are in, restore must give every rank its
            heads back, and a chunk whose second part never arrives must stay invisible.
``health``  three ranks with a :class:`PeerMonitor`: rank 2 leaves in an orderly way after
            step 1, rank 1 exits without a word after step 2; rank 0 must learn of both on the
            host, before its next step.
``serve``   the leader / follower layer that puts a tensor-parallel engine behind one HTTP front
            end: rank 0 announces every engine call, the other ranks replay it; all ranks must
            have executed the same calls with the same arguments, in the same order.
``serve_loop`` the engine loop on the leader over a real engine on every rank (concurrent requests,
            a cancellation, a chunk store between steps): followers must replay to the same tokens.
``pipeline`` every rank one pipeline stage of the oracle engine (layer ranges, per-stage store
            files, multi-part commits, activations over point-to-point sends); tokens and logits must
            equal those of a single process with all layers.
``late``    rank 0 alone of a two-rank world: the rendezvous must end with an error inside
            its time limit instead of waiting for ever.
"""

import asyncio
import datetime
import os
import sys
import tempfile
import threading
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from daser_b200.config import DaserConfig  # noqa: E402
from daser_b200.connector.core import ConnectorMeta, SchedulerHalf, TorchKVBackend, WorkerHalf  # noqa: E402
from daser_b200.connector.ipc_client import IPCClientSync  # noqa: E402
from daser_b200.kv.layout import KVGeometry, tp_head_range  # noqa: E402
from daser_b200.parallel.health import PeerLost, PeerMonitor  # noqa: E402


def _init(timeout_s: float = 60.0) -> tuple[int, int]:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank,
                            world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    return rank, world


def _bcast(obj, src=0):
    box = [obj]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def scenario_parts() -> int:
    rank, world = _init()
    L, H, D, B = 2, 4, 32, 16
    h0, hn = tp_head_range(H, world, rank)
    geo = KVGeometry(num_layers=L, num_kv_heads=hn, head_dim=D, block_tokens=B, dtype_bytes=2, codec="raw")
    tmp = _bcast(tempfile.mkdtemp(prefix="daser_gloo_") if rank == 0 else None)
    sock = f"{tmp}/d.sock"
    loop = plane = None
    if rank == 0:
        from daser_b200.server.__main__ import ControlPlane

        cfg = DaserConfig(store_path=f"{tmp}/unused.store", index_path="", total_slots=64, slot_size=geo.slot_size,
                          ipc_socket_path=sock)
        plane = ControlPlane(cfg)
        loop = asyncio.new_event_loop()
        ready = threading.Event()

        def serve():
            asyncio.set_event_loop(loop)
            loop.run_until_complete(plane.start())
            ready.set()
            loop.run_forever()

        threading.Thread(target=serve, daemon=True).start()
        ready.wait(20)
    dist.barrier()

    torch.manual_seed(7)  # same "model output" on every rank; each keeps its heads
    full = torch.randn(L, 8, 2, H, B, D).to(torch.bfloat16)
    pool = full[:, :, :, h0 : h0 + hn].clone()
    backend = TorchKVBackend(geo, pool, [1.0] * (D // 2))
    worker = WorkerHalf(sock, f"{tmp}/rank{rank}.store", geo, backend, io_backend="posix", staging_slots=8,
                        create_store_slots=64)
    worker.commit_parts = (rank, world)
    sched = SchedulerHalf(sock, B, "m") if rank == 0 else None
    probe = IPCClientSync(sock)
    ok = True

    # step 1: store a 3-block chunk from blocks 5,1,6
    tokens = list(range(100, 100 + 3 * B))
    if rank == 0:
        sched.reserve_chunk_store("r1", tokens, [5, 1, 6])
        meta = sched.build_connector_meta(["r1"])
    else:
        meta = None
    meta = _bcast(meta)
    assert isinstance(meta, ConnectorMeta) and len(meta.reqs_to_store) == 1
    key = meta.reqs_to_store[0].chunk_key
    worker.bind_connector_metadata(meta)
    if rank == 1:
        # rank 0 commits its part first; the chunk must still be invisible
        dist.barrier()
        ok = ok and probe.lookup_chunks([key], "m") == [None]
        worker.wait_for_save()
        dist.barrier()
    else:
        worker.wait_for_save()
        dist.barrier()
        dist.barrier()
    worker.clear_connector_metadata()
    ok = ok and probe.lookup_chunks([key], "m")[0] is not None

    # step 2: restore it into other blocks on every rank; each gets its own heads back
    if rank == 0:
        sched.plan_chunk_loads("r2", [(key, 0)])
        sched.assign_chunk_blocks("r2", [2, 3, 4])
        meta = sched.build_connector_meta(["r2"])
    meta = _bcast(meta if rank == 0 else None)
    pool[:, [2, 3, 4]] = 0
    worker.bind_connector_metadata(meta)
    worker.start_load_kv()
    worker.clear_connector_metadata()
    ok = ok and torch.equal(pool[:, [2, 3, 4]], full[:, [5, 1, 6]][:, :, :, h0 : h0 + hn])
    ok = ok and not worker.take_load_errors()

    # step 3: a chunk whose second part never arrives (rank 1 "crashed" between write and commit)
    tokens2 = list(range(500, 500 + B))
    if rank == 0:
        sched.reserve_chunk_store("r3", tokens2, [7])
        meta = sched.build_connector_meta(["r3"])
    meta = _bcast(meta if rank == 0 else None)
    key2 = meta.reqs_to_store[0].chunk_key
    if rank == 0:
        worker.bind_connector_metadata(meta)
        worker.wait_for_save()
        worker.clear_connector_metadata()
    dist.barrier()
    ok = ok and probe.lookup_chunks([key2], "m") == [None]

    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    worker.shutdown()
    probe.close()
    dist.barrier()
    if rank == 0:
        asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
        loop.call_soon_threadsafe(loop.stop)
        print("PARTS_OK" if all(flags) else f"PARTS_FAIL {flags}", flush=True)
    dist.destroy_process_group()
    return 0 if all(flags) else 1


def scenario_health() -> int:
    rank, world = _init()
    store = dist.distributed_c10d._get_default_store()
    mon = PeerMonitor(store, rank, world, timeout_s=1.5, interval_s=0.2)
    seen = []
    for step in range(6):
        try:
            mon.check()
        except PeerLost as exc:
            seen.append((step, exc.ranks))
            if exc.ranks == [1, 2]:
                break
        if rank == 2 and step == 1:
            mon.leave()  # between steps, nothing in flight
            os._exit(0)
        if rank == 1 and step == 2:
            os._exit(0)  # no notice at all
        time.sleep(0.2 if step < 3 else 1.0)  # a "step"
    mon.close()
    if rank == 0:
        first_left = next((s for s, r in seen if 2 in r), None)
        both = next((s for s, r in seen if r == [1, 2]), None)
        print(f"seen={seen}", flush=True)
        # rank 2 announces its exit after its own step 1; ranks run their steps only loosely in step
        good = first_left is not None and 1 <= first_left <= 4 and both is not None
        print("HEALTH_OK" if good else "HEALTH_FAIL", flush=True)
        os._exit(0 if good else 1)  # peers are gone: skip the collective teardown
    return 0


def scenario_serve() -> int:
    from daser_b200.service.tp_serving import TPLeaderEngine, follower_loop

    rank, world = _init()

    class Engine:
        class cfg:
            block_tokens = 16

        def __init__(self):
            self.calls = []

        def store_chunk(self, tokens):
            self.calls.append(("store", tuple(tokens)))
            return "key"

        def generate(self, chunks, query, max_new_tokens=1, **kw):
            self.calls.append(("generate", tuple(map(tuple, chunks)), tuple(query), max_new_tokens, tuple(sorted(kw.items()))))
            return len(self.calls)

        def warm_up(self, *a, **kw):
            self.calls.append(("warm_up", a, tuple(sorted(kw.items()))))

        def submit(self, req):
            self.calls.append(("submit", tuple(map(tuple, req.chunks)), tuple(req.query), req.max_new_tokens,
                               req.store_misses, req.temperature, req.seed, tuple(req.stop_token_ids),
                               req.top_k, req.top_p))
            return req

        def has_work(self):
            return False

        def step(self):
            self.calls.append(("step",))

        def abort(self, req_id):
            self.calls.append(("abort", req_id))
            return True

        def close(self):
            self.calls.append(("close",))

    eng = Engine()
    if rank == 0:
        lead = TPLeaderEngine(eng, _bcast)
        lead.warm_up(token_counts=(64,))
        assert lead.store_chunk(range(32)) == "key"
        lead.generate([list(range(16)), list(range(16, 48))], [1, 2, 3], max_new_tokens=4)
        lead.generate([], [9], max_new_tokens=1, store_misses=True)
        # a local observer is not announced (followers log the same call without it)
        lead.generate([], [8], max_new_tokens=2, on_token=lambda t: None)
        eng.calls[-1] = eng.calls[-1][:4] + ((),)
        # the iteration-level calls an engine loop makes
        from daser_b200.engine.request import RagRequest

        lead.submit(RagRequest([[5] * 16], [6, 7], 3, store_misses=True, temperature=0.5, seed=42,
                               stop_token_ids=(2,), top_k=40, top_p=0.9))
        lead.step()
        lead.step()
        lead.abort("req-7")
        lead.close()
        try:
            lead.store_chunk([1] * 16)
            refused = False
        except RuntimeError:
            refused = True
    else:
        steps = follower_loop(eng, _bcast)
        refused = steps == 9
    logs = [None] * world
    dist.all_gather_object(logs, (eng.calls, refused))
    good = all(log == logs[0][0] for log, _ in logs) and all(r for _, r in logs) and len(logs[0][0]) == 10
    if rank == 0:
        print("SERVE_OK" if good else f"SERVE_FAIL {logs}", flush=True)
    dist.destroy_process_group()
    return 0 if good else 1


def scenario_serve_loop() -> int:
    """The engine loop on the leader over real (oracle) engines on every rank: requests arrive from
    several threads, one is cancelled, a chunk is stored between steps.  Every follower must end up
    having served the same requests to the same tokens, with all blocks returned."""
    import random
    from concurrent.futures import ThreadPoolExecutor

    from daser_b200.engine.loop import EngineLoop
    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.models.llama import PRESETS
    from daser_b200.service.tp_serving import TPLeaderEngine, follower_loop

    rank, world = _init()
    cfg = PRESETS["toy"]
    geo = KVGeometry(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
    tmp = _bcast(tempfile.mkdtemp(prefix="daser_loop_") if rank == 0 else None)
    planes = [_start_plane(tmp, "cp", geo.slot_size)] if rank == 0 else []
    dist.barrier()
    # every rank is a whole replica here (the protocol under test does not care how a rank computes)
    eng = CpuRagEngine(cfg, f"{tmp}/cp.sock", f"{tmp}/r{rank}.store", num_blocks=24, io_backend="posix")
    served = []
    real_submit = eng.submit
    eng.submit = lambda req: served.append(req) or real_submit(req)
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(20 + 7 * i)] for i in range(5)]
    if rank == 0:
        loop = EngineLoop(TPLeaderEngine(eng, _bcast))
        with ThreadPoolExecutor(5) as pool:
            futs = list(pool.map(lambda p: loop.submit([], p, 12, temperature=0.9, seed=len(p)), prompts))
        long_one = loop.submit([], prompts[0], 200)
        loop.call("store_chunk", list(range(32))).result(60)
        time.sleep(0.2)
        loop.cancel(long_one)
        done = [f.result(120) for f in futs]
        try:
            long_one.result(60)
            cancelled = False
        except RuntimeError:
            cancelled = True
        loop.close()
        loop.engine.close()                                   # tells the followers to stop
        ok = cancelled and all(len(r.generated) == 12 for r in done)
    else:
        follower_loop(eng, _bcast)
        ok = True
    mine = sorted((r.req_id, tuple(r.generated) if r.error is None else r.error) for r in served)
    # the cancelled request stops at a step that is the same on every rank
    ok = ok and eng.blocks.num_free == 24 and not eng.has_work()
    logs = [None] * world
    dist.all_gather_object(logs, (mine, bool(ok)))
    good = all(o for _, o in logs) and all(m == logs[0][0] for m, _ in logs) and len(logs[0][0]) == 6
    if rank == 0:
        for plane, lp in planes:
            asyncio.run_coroutine_threadsafe(plane.stop(save=False), lp).result(10)
            lp.call_soon_threadsafe(lp.stop)
        print("SERVE_LOOP_OK" if good else f"SERVE_LOOP_FAIL {logs}", flush=True)
    dist.destroy_process_group()
    return 0 if good else 1


def scenario_late() -> int:
    t0 = time.time()
    try:
        _init(timeout_s=3.0)
    except Exception as exc:  # DistStoreError / DistNetworkError / RuntimeError by version
        print(f"RENDEZVOUS_FAILED after {time.time() - t0:.1f}s: {type(exc).__name__}", flush=True)
        return 7
    print("RENDEZVOUS_UNEXPECTEDLY_OK", flush=True)
    return 1


def _start_plane(tmp: str, name: str, slot_size: int, position=None):
    from daser_b200.server.__main__ import ControlPlane

    cfg = DaserConfig(store_path=f"{tmp}/{name}.unused", index_path="", total_slots=256, slot_size=slot_size,
                      ipc_socket_path=f"{tmp}/{name}.sock")
    plane = ControlPlane(cfg, position_encoder=position)
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


def scenario_pipeline() -> int:
    """Every rank is one pipeline stage of the oracle engine (5 layers over WORLD_SIZE stages, so
    the split is uneven); rank 0 also runs the control plane, and a lone single-process engine on
    a control plane of its own to compare with."""
    import dataclasses
    import random

    from daser_b200.engine.rag_cpu import CpuRagEngine
    from daser_b200.models.llama import PRESETS
    from daser_b200.parallel.pp import PipelineCpuEngine, partition_layers, stage_geometry
    from daser_b200.position import RopeReencoder

    rank, world = _init()
    cfg = dataclasses.replace(PRESETS["toy"], num_layers=5)
    tmp = _bcast(tempfile.mkdtemp(prefix="daser_pp_") if rank == 0 else None)
    geo = stage_geometry(cfg, world)
    planes = []
    if rank == 0:
        planes.append(_start_plane(tmp, "pp", geo.slot_size, RopeReencoder(cfg.head_dim, cfg.rope_theta)))
    dist.barrier()
    eng = PipelineCpuEngine(cfg, f"{tmp}/pp.sock", f"{tmp}/pp.store", num_blocks=128, io_backend="posix")
    ok = eng.layers == partition_layers(5, world)[rank] and geo.num_layers == -(-5 // world)
    rng = random.Random(4)
    chunks = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (32, 48, 32)]
    query = [rng.randrange(cfg.vocab_size) for _ in range(7)]
    probe = IPCClientSync(f"{tmp}/pp.sock")

    keys = [eng.store_chunk(c) for c in chunks[:2]]                      # chunk 2 stays unknown: computed
    ok = ok and all(m is not None for m in probe.lookup_chunks(keys, "default"))
    res = eng.run_request([], [chunks[1], chunks[2], chunks[0]], query)   # restored, computed, restored
    ok = ok and res.restored == [True, False, True]
    ok = ok and (res.logits is not None) == (rank == world - 1)
    gen = eng.generate([chunks[1], chunks[0]], query, max_new_tokens=4)
    ok = ok and gen.restored_chunks == 2 and len(gen.generated) == 4

    if rank == 0:
        # the same calls on one process with all layers
        from daser_b200.kv.layout import KVGeometry as G

        g1 = G(cfg.num_layers, cfg.num_kv_heads, cfg.head_dim, cfg.block_tokens, 4, "raw")
        planes.append(_start_plane(tmp, "one", g1.slot_size, RopeReencoder(cfg.head_dim, cfg.rope_theta)))
        lone = CpuRagEngine(cfg, f"{tmp}/one.sock", f"{tmp}/one.store", num_blocks=128, io_backend="posix")
        for c in chunks[:2]:
            lone.store_chunk(c)
        want = lone.run_request([], [chunks[1], chunks[2], chunks[0]], query)
        want_gen = lone.generate([chunks[1], chunks[0]], query, max_new_tokens=4)
        lone.close()
        ok = ok and want_gen.generated == gen.generated
        want_logits = want.logits
    else:
        want_logits = None
    want_logits = _bcast(want_logits)
    if rank == world - 1:
        err = (res.logits - want_logits).abs().max().item()
        print(f"pipeline logits max abs diff {err:.2e}", flush=True)
        ok = ok and err < 1e-3

    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    eng.close()
    probe.close()
    dist.barrier()
    for plane, loop in planes:
        asyncio.run_coroutine_threadsafe(plane.stop(save=False), loop).result(10)
        loop.call_soon_threadsafe(loop.stop)
    if rank == 0:
        print("PIPELINE_OK" if all(flags) else f"PIPELINE_FAIL {flags}", flush=True)
    return 0 if all(flags) else 1


if __name__ == "__main__":
    sys.exit({"parts": scenario_parts, "health": scenario_health, "serve": scenario_serve,
              "late": scenario_late, "pipeline": scenario_pipeline, "serve_loop": scenario_serve_loop}[sys.argv[1]]())
