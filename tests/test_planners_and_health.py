"""Host-side planning helpers and the peer monitor, in process (no GPU, no child processes)."""

import time

import pytest
import torch
import torch.distributed as dist

from daser_b200.models.llama import PRESETS, LlamaWeights, shard_weights
from daser_b200.ops import attention, gemm
from daser_b200.parallel.health import PeerLost, PeerMonitor


def test_split_plans_cover_the_context_and_respect_the_scratch_limit():
    for seqs, hkv, qlen, group, ctx in [(1, 8, 64, 8, 3328), (1, 1, 64, 8, 3261), (64, 8, 1, 8, 32768),
                                        (4, 2, 7, 4, 100), (1, 8, 256, 8, 8192), (1, 4, 130, 1, 513)]:
        nsplit, split_tokens = attention.plan_splits(seqs, hkv, qlen, group, ctx, 16)
        assert nsplit >= 1 and split_tokens % 16 == 0
        assert nsplit * split_tokens >= ctx > (nsplit - 1) * split_tokens
        rows = seqs * qlen * hkv * group
        n2, _ = attention.plan_splits(seqs, hkv, qlen, group, ctx, 16, rows=rows)
        assert n2 * rows <= max(attention.MAX_ROW_SPLITS, rows)
    # chunked prefill goes to 128-row CTAs with key tiles of 64: whole tiles per split
    nsplit, split_tokens = attention.plan_splits(1, 8, 64, 8, 3328, 16)
    assert split_tokens % attention.TC_KEY_TILE == 0 and nsplit > 1


def test_gemm_plans_and_swiglu_fusion_rule():
    assert gemm.plan_tiles(8192, 8192, 8192) == (256, 1)
    bn, ks = gemm.plan_tiles(64, 8192, 8192)
    assert bn == 128 and ks > 1  # few tiles: split K to fill the GPU
    assert gemm.plan_tiles(64, 57344, 8192) == (128, 1)
    assert gemm.can_fuse_swiglu(64, 57344, 8192)        # TP=1 gate/up of Llama-3-70B
    assert not gemm.can_fuse_swiglu(64, 7168, 8192)     # TP=8 shard: split-K, activation stays a kernel
    assert gemm.expected_arrivals(64, 8192, 64, 1, 8, 8, 1024) == [128] * 8


def test_gate_up_interleave_roundtrip_and_sharding_rule():
    cfg = PRESETS["tiny-gqa"]
    w = LlamaWeights.random(cfg, "cpu", torch.float32, seed=1)
    plain = w.layers[0].w_gate_up.clone()
    shard = shard_weights(w, 2, 1)
    w.interleave_gate_up_()
    assert w.gate_up_block == 64
    il = w.layers[0].w_gate_up
    assert torch.equal(il[:64], plain[:64]) and torch.equal(il[64:128], plain[cfg.intermediate : cfg.intermediate + 64])
    assert torch.equal(w.gate_up_plain(w.layers[0]), plain)
    assert torch.equal(gemm.interleave_gate_up(plain), il)
    w.interleave_gate_up_()  # idempotent
    with pytest.raises(AssertionError):
        shard_weights(w, 2, 0)  # shard the plain layout, then interleave the shard
    shard.interleave_gate_up_()
    inter = cfg.intermediate // 2
    assert torch.equal(shard.gate_up_plain(shard.layers[0])[:inter], plain[inter : 2 * inter])


def test_peer_monitor_leave_and_missed_heartbeats():
    store = dist.HashStore()
    a = PeerMonitor(store, 0, 3, timeout_s=0.3, interval_s=0.05, start=False)
    b = PeerMonitor(store, 1, 3, timeout_s=0.3, interval_s=0.05, start=False)
    c = PeerMonitor(store, 2, 3, timeout_s=0.3, interval_s=0.05, start=False)
    a.poll()
    a.check()  # everybody is there
    c.leave()
    with pytest.raises(PeerLost) as e:
        a.check()
    assert e.value.ranks == [2] and "left" in e.value.why
    # rank 1 keeps beating for a while, then stops without a word
    for _ in range(3):
        b._beat()
        a.poll()
        time.sleep(0.05)
    assert a.lost() == [2]
    time.sleep(0.4)
    a.poll()
    with pytest.raises(PeerLost) as e:
        a.check()
    assert e.value.ranks == [1, 2] and "heartbeat" in e.value.why
    for m in (a, b, c):
        m.close()


def test_peer_monitor_single_rank_is_a_no_op():
    m = PeerMonitor(dist.HashStore(), 0, 1)
    m.check()
    m.leave()
    m.close()


def test_pipeline_partition_and_stage_geometry():
    from daser_b200.models.llama import PRESETS
    from daser_b200.parallel.pp import partition_layers, stage_geometry, stage_store_path

    assert partition_layers(80, 8) == [range(10 * i, 10 * i + 10) for i in range(8)]
    parts = partition_layers(36, 5)                          # Qwen3-8B over five stages: 8, 7, 7, 7, 7
    assert [len(p) for p in parts] == [8, 7, 7, 7, 7] and parts[0].start == 0 and parts[-1].stop == 36
    assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
    for bad in (0, 37):
        with pytest.raises(ValueError):
            partition_layers(36, bad)
    cfg = PRESETS["qwen3-8b"]
    geo = stage_geometry(cfg, 5, dtype_bytes=2)
    assert geo.num_layers == 8 and geo.slot_size == 8 * 2 * 16 * 8 * 128 * 2    # the widest stage sizes the slots
    assert stage_store_path("/mnt/kv/daser.store", 2, 5) == "/mnt/kv/daser.store.pp2of5"


def test_row_buckets_are_few_idempotent_and_never_smaller_than_the_step():
    from daser_b200.engine.runner import GpuModelRunner

    b = GpuModelRunner.bucket_rows
    assert [b(n) for n in (1, 5, 16)] == [1, 5, 16]              # decode batches, prompt tails: exact
    assert [b(n) for n in (17, 64, 65, 128)] == [32, 64, 80, 128]
    assert [b(n) for n in (129, 303, 512, 513, 1000)] == [192, 320, 512, 640, 1024]
    for n in range(1, 2049):
        assert b(n) >= n and b(b(n)) == b(n)
        assert b(n) - n < (16 if n <= 128 else 64 if n <= 512 else 128)
    assert len({b(n) for n in range(1, 1025)}) <= 16 + 7 + 6 + 4  # the graphs a runner can end up holding
