"""The vLLM adapter driven by a fake engine: hooks are called in vLLM's order with CPU tensors.

The reference has no unit coverage of these hooks (they only run under a GPU integration
test); here a cold pass stores a prompt's KV and a warm pass restores it, for both KV layouts
vLLM uses.
"""

from types import SimpleNamespace

import pytest
import torch

from conftest import LiveControlPlane

pytest.importorskip("vllm.distributed.kv_transfer.kv_connector.v1.base")
pytestmark = pytest.mark.slow

L, NB, B, H, D = 3, 12, 16, 2, 32


def _vllm_config(lp, **extra):
    cfg = {"socket_path": lp.socket_path, "store_path": lp.cfg.store_path, "block_tokens": B, **extra}
    return SimpleNamespace(kv_transfer_config=SimpleNamespace(kv_connector_extra_config=cfg),
                           parallel_config=SimpleNamespace(tensor_parallel_size=1, rank=0))


def _caches(layout, seed):
    """Evenly spaced per-layer views of one cross-layer allocation."""
    g = torch.Generator().manual_seed(seed)
    shape = (2, NB, B, H, D) if layout == "KNTHD" else (NB, 2, B, H, D)
    big = torch.randn((L, *shape), generator=g).to(torch.bfloat16)
    return {f"model.layers.{i}.attn": big[i] for i in range(L)}, big


def _request(rid, tokens):
    return SimpleNamespace(request_id=rid, prompt_token_ids=tokens)


def _blocks(ids):
    return SimpleNamespace(get_block_ids=lambda: (ids,))


@pytest.mark.parametrize("layout", ["KNTHD", "NKTHD"])
@pytest.mark.parametrize("codec_name", ["raw", "fp8b16"])
def test_cold_store_then_warm_load(tmp_path, layout, codec_name):
    from daser_b200.connector.daser_connector import DaserConnector, DaserConnectorMeta, describe_kv_caches
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole

    bytes_per = 2 if codec_name == "raw" else 1.25
    slot = int(L * 2 * B * H * D * bytes_per)
    lp = LiveControlPlane(tmp_path, total_slots=32, slot_size=slot).start()
    cfg = _vllm_config(lp, codec=codec_name)
    sched = DaserConnector(cfg, KVConnectorRole.SCHEDULER)
    worker = DaserConnector(cfg, KVConnectorRole.WORKER)
    try:
        caches, big = _caches(layout, 1)
        assert describe_kv_caches(caches)["layout"] == layout
        worker.register_kv_caches(caches)
        tokens = list(range(100, 100 + 50))  # 3 full blocks + 2 tokens
        # ---- cold pass: miss -> reservation -> store ----
        req = _request("r1", tokens)
        assert sched.get_num_new_matched_tokens(req, 0) == (0, False)
        assert sched.get_num_new_matched_tokens(req, 0) == (0, False)  # vLLM may ask twice
        sched.update_state_after_alloc(req, _blocks([7, 2, 9, 4]), 0)
        meta = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r1": 50}))
        assert isinstance(meta, DaserConnectorMeta) and len(meta.reqs_to_store) == 1
        assert meta.reqs_to_store[0].block_ids == [7, 2, 9]
        worker.bind_connector_metadata(meta)
        worker.start_load_kv(None)
        for name in caches:
            worker.save_kv_layer(name, caches[name], None)
        worker.get_kv_connector_stats()  # start a fresh interval
        worker.wait_for_save()
        worker.clear_connector_metadata()
        stats = worker.get_kv_connector_stats()
        assert stats is not None and stats.data["bytes_stored"] == 3 * slot and not stats.is_empty()
        assert worker.get_kv_connector_stats() is None  # nothing moved since
        assert sched.request_finished(req, [7, 2, 9, 4]) == (False, None)
        # ---- warm pass in a fresh engine: hit -> load into other blocks ----
        caches2, big2 = _caches(layout, 2)
        worker2 = DaserConnector(cfg, KVConnectorRole.WORKER)
        worker2.register_kv_caches(caches2)
        req2 = _request("r2", tokens + [1, 2, 3])
        n, is_async = sched.get_num_new_matched_tokens(req2, 0)
        assert (n, is_async) == (48, False)
        sched.update_state_after_alloc(req2, _blocks([1, 5, 3, 8]), 48)
        meta2 = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r2": 5}))
        assert meta2.reqs_to_load[0].block_ids == [1, 5, 3] and not meta2.reqs_to_store
        worker2.bind_connector_metadata(meta2)
        worker2.start_load_kv(None)
        worker2.wait_for_save()
        worker2.clear_connector_metadata()
        assert worker2.get_block_ids_with_load_errors() == set()
        axis = 2 if layout == "KNTHD" else 1  # block axis of the stacked [L, ...] tensor
        for src, dst in zip([7, 2, 9], [1, 5, 3]):
            want = big.select(axis, src).float()
            got = torch.stack([caches2[n] for n in caches2]).select(axis, dst).float()
            if codec_name == "raw":
                assert torch.equal(got, want)
            else:
                assert torch.allclose(got, want, atol=0.3, rtol=0.13)
        untouched = torch.stack([caches2[n] for n in caches2]).select(axis, 8)
        assert torch.equal(untouched, big2.select(axis, 8))
        worker2.shutdown()
    finally:
        worker.shutdown()
        sched.shutdown()
        lp.stop()


def test_partial_commits_publish_only_when_every_rank_arrived(tmp_path):
    from daser_b200.connector.ipc_client import IPCClientSync

    lp = LiveControlPlane(tmp_path).start()
    try:
        c = IPCClientSync(lp.socket_path)
        c.alloc_chunk("k", 16, "default")
        c.commit_chunk("k", part=0, parts=2)
        assert c.lookup_chunks(["k"], "default") == [None]
        c.commit_chunk("k", part=0, parts=2)  # a repeat does not count twice
        assert c.lookup_chunks(["k"], "default") == [None]
        c.commit_chunk("k", part=1, parts=2)
        assert c.lookup_chunks(["k"], "default")[0]["chunk_key"] == "k"
        c.close()
    finally:
        lp.stop()


def test_vllm_factory_resolves_the_connector_by_module_path():
    """What `vllm serve --kv-transfer-config '{"kv_connector": "DaserConnector",
    "kv_connector_module_path": "daser_b200.connector.daser_connector", ...}'` does first."""
    pytest.importorskip("vllm")
    from vllm.config import KVTransferConfig
    from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1

    from daser_b200.connector.daser_connector import DaserConnector

    ktc = KVTransferConfig(kv_connector="DaserConnector", kv_role="kv_both",
                           kv_connector_module_path="daser_b200.connector.daser_connector",
                           kv_connector_extra_config={"socket_path": "/tmp/x.sock", "block_tokens": 16})
    cls = KVConnectorFactory.get_connector_class(ktc)
    assert cls is DaserConnector and issubclass(cls, KVConnectorBase_V1)
    # every abstract hook of the installed vLLM's base class is implemented
    assert not getattr(cls, "__abstractmethods__", None)


class _FlashAttnLike:
    """The stride-order hook of vLLM's FlashAttention backend (per-layer shape (2, N, T, H, D))."""

    order = (2, 0, 1, 3, 4, 5)  # NHD: physical (blocks, layers, 2, block, heads, dim)

    @classmethod
    def get_kv_cache_stride_order(cls, include_num_layers_dimension=False):
        assert include_num_layers_dimension
        return cls.order


class _FlashAttnLikeHND(_FlashAttnLike):
    order = (2, 4, 0, 1, 3, 5)  # HND: physical (blocks, heads, layers, 2, block, dim)


@pytest.mark.parametrize("backend", [_FlashAttnLike, _FlashAttnLikeHND])
def test_cross_layer_tensor_registration_store_and_load(tmp_path, backend):
    """vLLM answers prefer_cross_layer_blocks with ONE tensor in physical order and calls
    register_cross_layers_kv_cache instead of register_kv_caches."""
    from daser_b200.connector.daser_connector import DaserConnector
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole

    slot = L * 2 * B * H * D * 2
    lp = LiveControlPlane(tmp_path, total_slots=32, slot_size=slot).start()
    cfg = _vllm_config(lp)
    sched = DaserConnector(cfg, KVConnectorRole.SCHEDULER)

    def physical(seed):
        g = torch.Generator().manual_seed(seed)
        logical_shape = (L, 2, NB, B, H, D)
        phys_shape = tuple(logical_shape[i] for i in backend.order)
        return torch.randn(phys_shape, generator=g).to(torch.bfloat16)

    def logical(t):  # (L, 2, N, T, H, D) view of the physical tensor
        return t.permute(*[backend.order.index(i) for i in range(6)])

    worker = DaserConnector(cfg, KVConnectorRole.WORKER)
    worker2 = DaserConnector(cfg, KVConnectorRole.WORKER)
    try:
        assert worker.prefer_cross_layer_blocks
        cache1 = physical(1)
        worker.register_cross_layers_kv_cache(cache1, backend)
        tokens = list(range(200, 200 + 48))
        req = _request("r1", tokens + [5])
        assert sched.get_num_new_matched_tokens(req, 0) == (0, False)
        sched.update_state_after_alloc(req, _blocks([7, 2, 9, 4]), 0)
        meta = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r1": 49}))
        worker.bind_connector_metadata(meta)
        worker.start_load_kv(None)
        worker.wait_for_save()
        worker.clear_connector_metadata()
        sched.request_finished(req, [7, 2, 9, 4])

        cache2 = physical(2)
        before = cache2.clone()
        worker2.register_cross_layers_kv_cache(cache2, backend)
        req2 = _request("r2", tokens + [1, 2, 3])
        assert sched.get_num_new_matched_tokens(req2, 0) == (48, False)
        sched.update_state_after_alloc(req2, _blocks([1, 5, 3, 8]), 48)
        meta2 = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r2": 3}))
        worker2.bind_connector_metadata(meta2)
        worker2.start_load_kv(None)
        worker2.clear_connector_metadata()
        assert worker2.get_block_ids_with_load_errors() == set()
        for src, dst in zip([7, 2, 9], [1, 5, 3]):
            assert torch.equal(logical(cache2)[:, :, dst], logical(cache1)[:, :, src])
        assert torch.equal(logical(cache2)[:, :, 8], logical(before)[:, :, 8])
        assert worker2.reset_cache() is True
    finally:
        worker.shutdown()
        worker2.shutdown()
        sched.shutdown()
        lp.stop()


def test_connector_stats_container():
    from daser_b200.connector.daser_connector import DaserConnector, DaserKVConnectorStats

    a = DaserConnector.build_kv_connector_stats({"bytes_loaded": 10, "load_errors": 0})
    b = DaserKVConnectorStats(data={"bytes_loaded": 5, "bytes_stored": 7})
    assert not a.is_empty() and DaserConnector.build_kv_connector_stats().is_empty()
    assert a.aggregate(b).reduce() == {"bytes_loaded": 15, "load_errors": 0, "bytes_stored": 7}
    a.reset()
    assert a.is_empty()


def test_prometheus_metrics_hook_counts_per_engine():
    """vLLM's logger process builds the connector's Prometheus metrics once and feeds it the reduced
    stats of every interval: counters per field, labelled per engine."""
    from types import SimpleNamespace

    from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram

    from daser_b200.connector.daser_connector import DaserConnector

    reg = CollectorRegistry()

    def bound(cls):
        return lambda **kw: cls(registry=reg, **kw)

    prom = DaserConnector.build_prom_metrics(
        SimpleNamespace(kv_transfer_config=None), {Gauge: bound(Gauge), Counter: bound(Counter), Histogram: bound(Histogram)},
        ["model_name", "engine"], {0: ["toy", "0"], 1: ["toy", "1"]})
    assert prom is not None
    prom.observe({"bytes_loaded": 100, "bytes_stored": 0, "load_errors": 2, "unknown_field": 5}, engine_idx=0)
    prom.observe({"bytes_loaded": 50}, engine_idx=0)
    prom.observe({"bytes_loaded": 7}, engine_idx=1)
    get = lambda name, eng: reg.get_sample_value(name, {"model_name": "toy", "engine": eng})  # noqa: E731
    assert get("vllm:daser_bytes_loaded_total", "0") == 150 and get("vllm:daser_bytes_loaded_total", "1") == 7
    assert get("vllm:daser_load_errors_total", "0") == 2
    assert get("vllm:daser_bytes_stored_total", "0") is None   # nothing stored: no child yet
