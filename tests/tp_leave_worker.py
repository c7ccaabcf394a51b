"""Worker of the peer-loss GPU test: run with ``torch.distributed.run --nproc-per-node 2``.

Both ranks run one fused tensor-parallel forward.  Then rank 1 leaves in an orderly way: its
stream is drained, it tells the group through the store, and it exits; nothing of its is in
flight.  Rank 0 must learn of it on the host at its next ``check_peers`` -- before it launches
anything that would wait for rank 1 -- and its GPU context must still be usable.  The test is
run with NVLS off and no multicast mapping on the symmetric buffers; if the buffers turn out to
have one anyway, nobody leaves and the worker reports ``TP_LEAVE_SKIPPED``.
"""

import os
import random
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from daser_b200.engine.runner import GpuModelRunner, make_step_inputs  # noqa: E402
from daser_b200.models.llama import PRESETS, LlamaWeights, shard_weights  # noqa: E402
from daser_b200.ops import elementwise as ew  # noqa: E402
from daser_b200.parallel.health import PeerLost  # noqa: E402
from daser_b200.parallel.tp import TPContext  # noqa: E402


def main() -> None:
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tp = dist.get_world_size()
    cfg = PRESETS["tiny-gqa"]
    full = LlamaWeights.random(cfg, "cuda", torch.bfloat16, seed=5, std=0.05)
    ctx = TPContext(cfg, dist.group.WORLD, max_tokens=128)
    runner = GpuModelRunner(cfg, shard_weights(full, tp, rank), 64, 128, 8, ctx)
    rng = random.Random(0)
    tokens = [rng.randrange(cfg.vocab_size) for _ in range(33)]
    inp = make_step_inputs([{"tokens": tokens, "start_pos": 0, "block_table": [3, 7, 1]}], 16, "cuda")
    ctx.check_peers()
    first = int(runner.forward(inp)[0].item())
    runner.check_status()
    torch.cuda.synchronize()
    ctx.barrier()
    torch.cuda.synchronize()

    bound = ctx.multicast_bound()
    flags = [None] * tp
    dist.all_gather_object(flags, bound, group=ctx._cpu_group)
    if any(flags):
        ctx.close()
        ctx.barrier()
        if rank == 0:
            print("TP_LEAVE_SKIPPED multicast mapping present", flush=True)
        dist.destroy_process_group()
        return

    if rank == 1:
        ctx.leave()  # drains this rank's stream, then tells the group
        print("rank 1 left", flush=True)
        os._exit(0)

    # rank 0: the next step must not be launched
    t0 = time.time()
    lost = None
    while time.time() - t0 < 20:
        try:
            ctx.check_peers()
        except PeerLost as exc:
            lost = exc.ranks
            break
        time.sleep(0.05)
    ok = lost == [1]
    # the context is intact: a kernel of this package on local memory still runs and is right
    x = torch.randn(64, cfg.hidden, device="cuda").to(torch.bfloat16)
    w = torch.ones(cfg.hidden, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    ew.add_rmsnorm(x, w, out=out, eps=1e-5)
    torch.cuda.synchronize()
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    ok = ok and (out.float() - ref).abs().max().item() < 0.05
    print(f"first token {first}; lost={lost} after {time.time() - t0:.2f}s", flush=True)
    print("TP_LEAVE_OK" if ok else "TP_LEAVE_FAIL", flush=True)
    sys.stdout.flush()
    os._exit(0 if ok else 1)  # the peer is gone: no collective teardown


if __name__ == "__main__":
    main()
