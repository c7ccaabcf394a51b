"""The vLLM adapter's CUDA path: the engine's bf16 KV tensors (vLLM's layouts, on the device) are
saved and restored by the fused kernels through the adapter's hooks."""

from types import SimpleNamespace

import pytest
import torch

from conftest import LiveControlPlane

pytest.importorskip("vllm.distributed.kv_transfer.kv_connector.v1.base")
pytestmark = pytest.mark.gpu

L, NB, B, H, D = 3, 12, 16, 2, 64


def _cfg(lp, **extra):
    cfg = {"socket_path": lp.socket_path, "store_path": lp.cfg.store_path, "block_tokens": B, **extra}
    return SimpleNamespace(kv_transfer_config=SimpleNamespace(kv_connector_extra_config=cfg),
                           parallel_config=SimpleNamespace(tensor_parallel_size=1, rank=0))


class _NHD:
    """FlashAttention's cross-layer stride order: physical (blocks, layers, 2, block, heads, dim)."""

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension=False):
        return (2, 0, 1, 3, 4, 5)


def _engine_cache(kind, seed):
    """(register(worker), logical view [L, 2, N, T, H, D]) of a KV cache laid out as vLLM would."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    if kind == "cross":
        phys = torch.randn((NB, L, 2, B, H, D), generator=g, device="cuda").to(torch.bfloat16)
        logical = phys.permute(1, 2, 0, 3, 4, 5)
        return (lambda w: w.register_cross_layers_kv_cache(phys, _NHD)), logical
    if kind == "KNTHD":
        big = torch.randn((L, 2, NB, B, H, D), generator=g, device="cuda").to(torch.bfloat16)
        logical = big
    else:  # NKTHD (FlashInfer)
        big = torch.randn((L, NB, 2, B, H, D), generator=g, device="cuda").to(torch.bfloat16)
        logical = big.permute(0, 2, 1, 3, 4, 5)
    caches = {f"model.layers.{i}.attn": big[i] for i in range(L)}
    return (lambda w: w.register_kv_caches(caches)), logical


@pytest.mark.parametrize("kind", ["KNTHD", "NKTHD", "cross"])
@pytest.mark.parametrize("codec_name", ["raw", "fp8b16"])
def test_cold_store_then_warm_load_on_the_device(tmp_path, kind, codec_name):
    from daser_b200.connector.daser_connector import DaserConnector
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole

    slot = int(L * 2 * B * H * D * (2 if codec_name == "raw" else 1.25))
    lp = LiveControlPlane(tmp_path, total_slots=32, slot_size=slot).start()
    cfg = _cfg(lp, codec=codec_name)
    sched = DaserConnector(cfg, KVConnectorRole.SCHEDULER)
    worker = DaserConnector(cfg, KVConnectorRole.WORKER)
    worker2 = DaserConnector(cfg, KVConnectorRole.WORKER)
    try:
        register, src = _engine_cache(kind, 1)
        register(worker)
        tokens = list(range(100, 100 + 50))  # 3 full blocks + 2 tokens
        req = SimpleNamespace(request_id="r1", prompt_token_ids=tokens)
        assert sched.get_num_new_matched_tokens(req, 0) == (0, False)
        sched.update_state_after_alloc(req, SimpleNamespace(get_block_ids=lambda: ([7, 2, 9, 4],)), 0)
        meta = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r1": 50}))
        worker.bind_connector_metadata(meta)
        worker.start_load_kv(None)
        worker.wait_for_save()
        worker.clear_connector_metadata()
        sched.request_finished(req, [7, 2, 9, 4])

        register2, dst = _engine_cache(kind, 2)
        before = dst.clone()
        register2(worker2)
        req2 = SimpleNamespace(request_id="r2", prompt_token_ids=tokens + [1, 2, 3])
        assert sched.get_num_new_matched_tokens(req2, 0) == (48, False)
        sched.update_state_after_alloc(req2, SimpleNamespace(get_block_ids=lambda: ([1, 5, 3, 8],)), 48)
        meta2 = sched.build_connector_meta(SimpleNamespace(num_scheduled_tokens={"r2": 5}))
        worker2.bind_connector_metadata(meta2)
        worker2.start_load_kv(None)
        worker2.clear_connector_metadata()
        torch.cuda.synchronize()
        assert worker2.get_block_ids_with_load_errors() == set()
        for s, d in zip([7, 2, 9], [1, 5, 3]):
            want, got = src[:, :, s].float(), dst[:, :, d].float()
            if codec_name == "raw":
                assert torch.equal(got, want)
            else:
                assert torch.allclose(got, want, atol=0.3, rtol=0.13)
        for untouched in (0, 8, 11):
            assert torch.equal(dst[:, :, untouched], before[:, :, untouched])
    finally:
        worker.shutdown()
        worker2.shutdown()
        sched.shutdown()
        lp.stop()
