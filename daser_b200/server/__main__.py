"""``python -m daser_b200.server`` — stand-alone control plane.

Capability parity: ``daser/server/__main__.py:25-182`` — the same flags
(``--store-path`` required, ``--store-size`` 10 GiB, ``--socket-path``,
``--index-path``, ``--slot-size`` 2 MiB with 0 meaning "derive",
``--block-tokens``, ``--num-kv-heads/--head-dim/--num-layers``,
``--dtype-bytes``, ``--model-id``, ``--log-level``), the
``store_size % slot_size == 0`` check, snapshot restore with cold start on
failure, retrieval-index rebuild, SIGTERM/SIGINT shutdown with a final
snapshot.

Added flags: ``--codec``, ``--position`` (``fixed`` or ``rope``),
``--rope-theta``, ``--snapshot-interval`` (periodic atomic snapshots; the
reference loses all metadata on a crash).
"""

from __future__ import annotations

import argparse
import asyncio
import os
import signal
from typing import Optional, Sequence

from daser_b200.config import CODECS, DaserConfig
from daser_b200.logging import init_logger
from daser_b200.position import FixedOffsetEncoder, PositionEncoder, RopeReencoder
from daser_b200.retrieval import ChunkOffsetIndex, RetrievalIndex
from daser_b200.server.chunk_manager import ChunkManager
from daser_b200.server.doc_registry import DocRegistry
from daser_b200.server.ipc_server import IPCServer
from daser_b200.server.metadata_store import MetadataStore

logger = init_logger(__name__)

_GIB = 1024**3
_DEFAULT_SLOT = 2 * 1024 * 1024


def _parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="daser_b200.server", description=__doc__)
    p.add_argument("--store-path", required=True)
    p.add_argument("--store-size", type=int, default=10 * _GIB)
    p.add_argument("--socket-path", default="/tmp/daser.sock")
    p.add_argument("--index-path", default="/tmp/daser.index")
    p.add_argument("--slot-size", type=int, default=_DEFAULT_SLOT)
    p.add_argument("--block-tokens", type=int, default=16)
    p.add_argument("--num-kv-heads", type=int, default=0)
    p.add_argument("--head-dim", type=int, default=0)
    p.add_argument("--num-layers", type=int, default=0)
    p.add_argument("--dtype-bytes", type=int, default=2)
    p.add_argument("--model-id", default="default")
    p.add_argument("--log-level", default="INFO")
    p.add_argument("--codec", choices=CODECS, default="raw")
    p.add_argument("--position", choices=("fixed", "rope"), default="fixed")
    p.add_argument("--rope-theta", type=float, default=10000.0)
    p.add_argument("--snapshot-interval", type=float, default=0.0)
    p.add_argument("--no-fast-lookup", action="store_true",
                   help="do not start the native thread that answers lookups by key on <socket>.fast")
    args = p.parse_args(argv)
    if args.no_fast_lookup:
        os.environ["DASER_FAST_LOOKUP"] = "0"
    return args


def _build_daser_config(args: argparse.Namespace) -> DaserConfig:
    cfg = DaserConfig(
        store_path=args.store_path,
        index_path=args.index_path,
        slot_size=args.slot_size,
        ipc_socket_path=args.socket_path,
        log_level=args.log_level,
        num_kv_heads=args.num_kv_heads,
        head_dim=args.head_dim,
        num_layers=args.num_layers,
        block_tokens=args.block_tokens,
        dtype_bytes=args.dtype_bytes,
        model_id=args.model_id,
        codec=getattr(args, "codec", "raw"),
        rope_theta=getattr(args, "rope_theta", 10000.0),
        snapshot_interval_s=getattr(args, "snapshot_interval", 0.0),
    )
    slot = cfg.resolved_slot_size()
    if args.store_size <= 0 or args.store_size % slot:
        raise ValueError(
            f"store_size={args.store_size} must be a positive multiple of "
            f"slot_size={slot}"
        )
    # slot_size stays as given (0 = derived from the model parameters, through
    # resolved_slot_size(), which is what every consumer calls): the reference's behaviour
    cfg.total_slots = args.store_size // slot
    return cfg


class ControlPlane:
    """Ring + metadata + registry + index + RPC server, wired once.

    Shared by this CLI, the service (which embeds it) and the tests.
    """

    def __init__(
        self,
        cfg: DaserConfig,
        retrieval_index: Optional[RetrievalIndex] = None,
        position_encoder: Optional[PositionEncoder] = None,
    ) -> None:
        self.cfg = cfg
        self.store = MetadataStore(cfg.total_slots)
        self.docs = DocRegistry()
        self.ring = ChunkManager(cfg.total_slots, self.store, self.docs)
        self.index = retrieval_index or ChunkOffsetIndex(cfg.block_tokens)
        self.position = position_encoder or FixedOffsetEncoder(0)
        self.server: Optional[IPCServer] = None
        self._snap_task: Optional[asyncio.Task] = None

    def restore(self) -> bool:
        """Load the snapshot if there is one; any failure means a cold start."""
        path = self.cfg.index_path
        if not path or not os.path.exists(path):
            return False
        try:
            self.ring.load(path)
        except Exception as exc:
            logger.warning("[SERVER] snapshot %s unusable (%r); cold start", path, exc)
            self.store = MetadataStore(self.cfg.total_slots)
            self.docs = DocRegistry()
            self.ring = ChunkManager(self.cfg.total_slots, self.store, self.docs)
            return False
        return True

    async def start(self) -> IPCServer:
        restored = self.restore()
        if restored:
            for meta in self.store.iter_chunks():
                if self.store.is_committed(meta.chunk_key):
                    await self.index.insert(meta)
                    anchor = self.store.anchor(meta.chunk_key)
                    if anchor and hasattr(self.index, "register_anchor"):
                        self.index.register_anchor(meta.chunk_key, anchor)  # scans find it after a restart
        geometry = {}
        try:
            geometry = self.cfg.geometry()
        except ValueError:
            pass
        self.server = IPCServer(
            self.cfg.ipc_socket_path,
            self.ring,
            self.index,
            self.position,
            slot_size=self.cfg.resolved_slot_size(),
            block_tokens=self.cfg.block_tokens,
            doc_registry=self.docs,
            geometry=geometry,
        )
        await self.server.start()
        if self.cfg.snapshot_interval_s > 0:
            self._snap_task = asyncio.create_task(self._periodic_snapshots())
        return self.server

    async def _periodic_snapshots(self) -> None:
        assert self.server is not None
        while True:
            await asyncio.sleep(self.cfg.snapshot_interval_s)
            if self.server.dirty:
                self.snapshot()

    def snapshot(self) -> None:
        if self.cfg.index_path:
            self.ring.save(self.cfg.index_path)
            if self.server is not None:
                self.server.clear_dirty()

    async def stop(self, save: bool = True) -> None:
        if self._snap_task is not None:
            self._snap_task.cancel()
            self._snap_task = None
        if save:
            try:
                self.snapshot()
            except OSError as exc:
                logger.error("[SERVER] final snapshot failed: %s", exc)
        if self.server is not None:
            await self.server.stop()
            self.server = None


def make_position_encoder(args: argparse.Namespace) -> PositionEncoder:
    if getattr(args, "position", "fixed") == "rope":
        return RopeReencoder(
            head_dim=args.head_dim or 128, theta=getattr(args, "rope_theta", 10000.0)
        )
    return FixedOffsetEncoder(0)


async def run_server(
    cfg: DaserConfig, position_encoder: Optional[PositionEncoder] = None
) -> None:
    init_logger("daser_b200", cfg.log_level)
    plane = ControlPlane(cfg, position_encoder=position_encoder)
    await plane.start()
    stop = asyncio.Event()
    loop = asyncio.get_running_loop()
    for sig in (signal.SIGTERM, signal.SIGINT):
        loop.add_signal_handler(sig, stop.set)
    logger.info(
        "[SERVER] ready: %d slots of %d bytes, socket %s",
        cfg.total_slots,
        cfg.resolved_slot_size(),
        cfg.ipc_socket_path,
    )
    await stop.wait()
    await plane.stop(save=True)


def main(argv: Optional[Sequence[str]] = None) -> None:
    args = _parse_args(argv)
    cfg = _build_daser_config(args)
    asyncio.run(run_server(cfg, make_position_encoder(args)))


if __name__ == "__main__":
    main()
