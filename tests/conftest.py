"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu``; everything else runs on CPU."""

import asyncio
import os
import sys
import threading

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        ndev = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        ndev = 0
    for item in items:
        if "gpu" in item.keywords and ndev < 1:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and ndev < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


class LiveControlPlane:
    """A real control plane on a temp socket, on its own thread and event loop."""

    def __init__(self, tmp_path, total_slots=64, slot_size=4096, block_tokens=16, position_encoder=None, **cfg_kw):
        from daser_b200.config import DaserConfig
        from daser_b200.server.__main__ import ControlPlane

        self.cfg = DaserConfig(
            store_path=str(tmp_path / "daser.store"),
            index_path=str(tmp_path / "daser.index"),
            total_slots=total_slots,
            slot_size=slot_size,
            ipc_socket_path=str(tmp_path / "d.sock"),
            block_tokens=block_tokens,
            **cfg_kw,
        )
        self.plane = ControlPlane(self.cfg, position_encoder=position_encoder)
        self.loop = asyncio.new_event_loop()
        self._ready = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        asyncio.set_event_loop(self.loop)
        self.loop.run_until_complete(self.plane.start())
        self._ready.set()
        self.loop.run_forever()

    def start(self):
        self.thread.start()
        assert self._ready.wait(10)
        return self

    def stop(self, save=False):
        fut = asyncio.run_coroutine_threadsafe(self.plane.stop(save=save), self.loop)
        fut.result(10)
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.thread.join(10)

    @property
    def socket_path(self):
        return self.cfg.ipc_socket_path


@pytest.fixture
def live_plane(tmp_path):
    lp = LiveControlPlane(tmp_path).start()
    yield lp
    lp.stop()
