"""vLLM ``KVConnectorBase_V1`` adapter.

Capability parity: ``daser/connector/daser_connector.py:115-710`` — the class vLLM loads
with ``kv_connector="DaserConnector"``,
``kv_connector_module_path="daser_b200.connector.daser_connector"``, ``kv_role="kv_both"``;
extra-config keys ``socket_path`` (``/tmp/daser.sock``), ``store_path``, ``slot_size`` (0 =
derive), ``block_tokens`` (16), ``model_id`` (``"default"``); scheduler-role hooks
``get_num_new_matched_tokens / update_state_after_alloc / build_connector_meta /
request_finished``; worker-role hooks ``register_kv_caches / bind_connector_metadata /
clear_connector_metadata / start_load_kv / wait_for_layer_load / save_kv_layer /
wait_for_save / shutdown``; ``hash_tokens``, ``ReqLoadSpec``, ``ReqStoreSpec`` and
``DaserConnectorMeta`` are importable from here.

The logic lives in :mod:`daser_b200.connector.core`; this file only translates vLLM objects.
Differences from the reference adapter:

* The KV layout is read from the registered tensors (FlashAttention ``(2, N, B, H, D)`` or
  FlashInfer ``(N, 2, B, H, D)``) and turned into explicit strides; the reference indexes
  ``kv[:, block_id]`` and breaks on the FlashInfer layout that compute capability 10.x selects.
* Additional extra-config keys: ``codec`` (``raw`` keeps the reference's container byte for
  byte, ``fp8b16`` compresses), ``io_backend``, ``hbm_slots``, ``host_slots``, ``staging_slots``
  (the pinned arena between the kernels and the file; longer chunks pass through it in pieces),
  ``write_behind`` (``wait_for_save`` returns with the file writes in flight; the chunk is committed
  when they are done, at the latest before the next load or save that needs the arena).
* Hooks the reference leaves at their defaults are implemented: ``register_cross_layers_kv_cache``,
  ``reset_cache``, ``get_block_ids_with_load_errors``,
  ``get_kv_connector_stats``, ``prefer_cross_layer_blocks``.
* Tensor parallel workers each keep their own store file (``<store_path>.tp<rank>``) holding
  their head slice, and a chunk becomes visible only after every rank has committed its part.
  The reference lets all ranks write the same offsets of one file.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from daser_b200.connector.core import (  # noqa: F401  (re-exported names of the reference module)
    ConnectorMeta,
    CudaKVBackend,
    ReqLoadSpec,
    ReqStoreSpec,
    SchedulerHalf,
    TorchKVBackend,
    WorkerHalf,
)
from daser_b200.hashing import hash_tokens  # noqa: F401
from daser_b200.kv.layout import KVGeometry
from daser_b200.logging import init_logger

try:  # vLLM is optional: the engine-agnostic core works without it
    from vllm.distributed.kv_transfer.kv_connector.v1.base import (
        KVConnectorBase_V1,
        KVConnectorMetadata,
        KVConnectorRole,
    )

    HAVE_VLLM = True
except Exception:  # pragma: no cover - exercised only where vLLM is absent
    HAVE_VLLM = False

    class KVConnectorMetadata:  # type: ignore[no-redef]
        pass

    class KVConnectorBase_V1:  # type: ignore[no-redef]
        def __init__(self, vllm_config=None, role=None, kv_cache_config=None):
            self._connector_metadata = None
            self._vllm_config = vllm_config
            self._role = role

        def bind_connector_metadata(self, connector_metadata):
            self._connector_metadata = connector_metadata

        def clear_connector_metadata(self):
            self._connector_metadata = None

    class KVConnectorRole:  # type: ignore[no-redef]
        SCHEDULER = "scheduler"
        WORKER = "worker"


logger = init_logger(__name__)


@dataclass
class DaserConnectorMeta(KVConnectorMetadata):
    """Per-step metadata carried from the scheduler process to every worker."""

    reqs_to_load: list[ReqLoadSpec] = field(default_factory=list)
    reqs_to_store: list[ReqStoreSpec] = field(default_factory=list)


def describe_kv_caches(kv_caches: dict[str, torch.Tensor]) -> dict[str, Any]:
    """Layout facts of vLLM's per-layer KV tensors.

    Returns ``layout`` (dimension letters per layer tensor: ``KNTHD`` for FlashAttention,
    ``NKTHD`` for FlashInfer), the layer stride in elements (layers must be evenly spaced in
    memory, e.g. one cross-layer allocation), block count, block size, heads and head dim.
    """
    names = list(kv_caches)
    first = kv_caches[names[0]]
    if first.dim() != 5:
        raise ValueError(f"expected 5-D KV tensors, got shape {tuple(first.shape)}")
    if first.shape[0] == 2 and first.shape[1] != 2:
        layout = "KNTHD"
    elif first.shape[1] == 2:
        layout = "NKTHD"
    else:
        raise ValueError(f"cannot tell K/V axis of KV tensor with shape {tuple(first.shape)}")
    dims = dict(zip(layout, first.shape))
    ptrs = [kv_caches[n].data_ptr() for n in names]
    stride_bytes = 0
    if len(ptrs) > 1:
        gaps = {b - a for a, b in zip(ptrs, ptrs[1:])}
        if len(gaps) != 1 or next(iter(gaps)) <= 0:
            raise ValueError(
                "KV layers are not evenly spaced in memory; enable cross-layer KV blocks "
                "(the connector asks for them through prefer_cross_layer_blocks)"
            )
        stride_bytes = next(iter(gaps))
    esize = first.element_size()
    if stride_bytes % esize:
        raise ValueError("layer stride is not a whole number of elements")
    return {
        "layout": layout, "layer_stride": stride_bytes // esize, "num_blocks": dims["N"], "block_tokens": dims["T"],
        "heads": dims["H"], "head_dim": dims["D"], "dtype": first.dtype, "names": names,
        "strides": dict(zip(layout, first.stride())),
    }


_STAT_KEYS = ("connector.bytes_loaded", "connector.bytes_stored", "connector.bytes_over_pcie",
              "connector.load_errors", "connector.store_errors")

try:  # vLLM's container for connector telemetry (worker -> logger process); absent in old versions
    from vllm.distributed.kv_transfer.kv_connector.v1.metrics import KVConnectorStats as _KVConnectorStats
except Exception:  # pragma: no cover
    _KVConnectorStats = None

if _KVConnectorStats is not None:
    from dataclasses import dataclass as _dataclass

    @_dataclass
    class DaserKVConnectorStats(_KVConnectorStats):  # type: ignore[misc,valid-type]
        """Byte and error counters of one interval; all fields are sums, so aggregation adds."""

        def reset(self) -> None:
            self.data = {}

        def aggregate(self, other: "DaserKVConnectorStats") -> "DaserKVConnectorStats":
            for k, v in other.data.items():
                self.data[k] = self.data.get(k, 0) + v
            return self

        def reduce(self) -> dict[str, int | float]:
            return dict(self.data)

        def is_empty(self) -> bool:
            return not any(self.data.values())
else:  # pragma: no cover
    DaserKVConnectorStats = None  # type: ignore[assignment,misc]

try:  # vLLM's hook for per-connector Prometheus metrics (logger process); absent in old versions
    from vllm.distributed.kv_transfer.kv_connector.v1.metrics import KVConnectorPromMetrics as _PromBase
except Exception:  # pragma: no cover
    _PromBase = None

_PROM_HELP = {
    "bytes_loaded": "Bytes of chunk KV restored into the paged cache",
    "bytes_stored": "Bytes of chunk KV written to the store",
    "bytes_over_pcie": "Bytes of chunk KV that crossed PCIe on the way in (store file or host tier)",
    "load_errors": "Blocks whose restore failed and were handed back to vLLM for recomputation",
    "store_errors": "Chunks whose write failed (left uncommitted)",
}

if _PromBase is not None:

    class DaserPromMetrics(_PromBase):  # type: ignore[misc,valid-type]
        """One counter per field of :class:`DaserKVConnectorStats`, labelled per engine:
        ``vllm:daser_<field>_total`` grows by what each stats interval reports."""

        def __init__(self, vllm_config: Any, metric_types: Any, labelnames: list[str],
                     per_engine_labelvalues: dict[int, list[object]]) -> None:
            super().__init__(vllm_config, metric_types, labelnames, per_engine_labelvalues)
            self._counters = {
                field: self._counter_cls(name=f"vllm:daser_{field}", documentation=doc, labelnames=labelnames)
                for field, doc in _PROM_HELP.items()
            }
            self._children: dict[tuple[int, str], Any] = {}

        def observe(self, transfer_stats_data: dict[str, Any], engine_idx: int = 0) -> None:
            for field, value in transfer_stats_data.items():
                counter = self._counters.get(field)
                if counter is None or not value or value < 0:
                    continue
                child = self._children.get((engine_idx, field))
                if child is None:
                    child = counter.labels(*self.per_engine_labelvalues[engine_idx])
                    self._children[(engine_idx, field)] = child
                child.inc(value)
else:  # pragma: no cover
    DaserPromMetrics = None  # type: ignore[assignment,misc]


class DaserConnector(KVConnectorBase_V1):
    def __init__(self, vllm_config: Any, role: Any, kv_cache_config: Any = None) -> None:
        try:
            super().__init__(vllm_config=vllm_config, role=role, kv_cache_config=kv_cache_config)
        except TypeError:  # older base classes take two arguments
            super().__init__(vllm_config=vllm_config, role=role)
        extra = dict(getattr(vllm_config.kv_transfer_config, "kv_connector_extra_config", None) or {})
        self._socket_path = extra.get("socket_path", "/tmp/daser.sock")
        self._store_path = extra.get("store_path", "/tmp/daser.store")
        self._slot_size = int(extra.get("slot_size", 0))
        self._block_tokens = int(extra.get("block_tokens", 16))
        self._model_id = extra.get("model_id", "default")
        self._codec = extra.get("codec", "raw")
        self._io_backend = extra.get("io_backend", "auto")
        self._hbm_slots = int(extra.get("hbm_slots", 0))
        self._host_slots = int(extra.get("host_slots", 0))
        self._staging_slots = int(extra.get("staging_slots", 256))
        self._write_behind = str(extra.get("write_behind", "0")).lower() in ("1", "true", "yes")
        par = getattr(vllm_config, "parallel_config", None)
        self._tp = int(getattr(par, "tensor_parallel_size", 1) or 1)
        self._rank = int(extra.get("tp_rank", getattr(par, "rank", 0) or 0)) % max(self._tp, 1)
        self._is_scheduler = role == KVConnectorRole.SCHEDULER
        self._sched: Optional[SchedulerHalf] = None
        self._worker: Optional[WorkerHalf] = None
        self._req_tokens: dict[str, int] = {}
        self._stats_seen: dict[str, float] = {}
        if self._is_scheduler:
            self._sched = SchedulerHalf(self._socket_path, self._block_tokens, self._model_id)

    # ------------------------------------------------------------------ class-level hints
    @property
    def prefer_cross_layer_blocks(self) -> bool:
        """One allocation holding every layer of a block matches the slot format exactly."""
        return True

    # ------------------------------------------------------------------ scheduler role
    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int) -> tuple[int, bool]:
        assert self._sched is not None
        tokens = list(request.prompt_token_ids)
        return self._sched.get_num_new_matched_tokens(request.request_id, tokens, num_computed_tokens)

    def update_state_after_alloc(self, request: Any, blocks: Any, num_external_tokens: int) -> None:
        assert self._sched is not None
        if hasattr(blocks, "get_block_ids"):
            block_ids = blocks.get_block_ids()[0]
        else:
            group0 = blocks.blocks[0]
            block_ids = [getattr(b, "block_id", b) for b in group0]
        self._sched.update_state_after_alloc(request.request_id, list(block_ids), num_external_tokens)

    def build_connector_meta(self, scheduler_output: Any) -> DaserConnectorMeta:
        assert self._sched is not None
        scheduled = list(getattr(scheduler_output, "num_scheduled_tokens", {}) or {})
        meta = self._sched.build_connector_meta(scheduled)
        return DaserConnectorMeta(meta.reqs_to_load, meta.reqs_to_store)

    def request_finished(self, request: Any, block_ids: list[int]) -> tuple[bool, Optional[dict[str, Any]]]:
        if self._sched is not None:
            self._sched.request_finished(request.request_id)
        return False, None

    # ------------------------------------------------------------------ worker role
    def register_cross_layers_kv_cache(self, kv_cache: torch.Tensor, attn_backend: Any) -> None:
        """vLLM's answer to ``prefer_cross_layer_blocks``: ONE tensor for all layers, handed over
        in its physical dimension order (FlashAttention: ``(blocks, layers, 2, block, heads, dim)``
        for the NHD layout, ``(blocks, heads, layers, 2, block, dim)`` for HND).  vLLM calls this
        INSTEAD of :meth:`register_kv_caches`.  The backend's stride order turns it back into
        per-layer views (strides kept), which is what the stride-driven registration consumes;
        with the NHD order a block's slot image is one contiguous run of the tensor."""
        try:
            order = tuple(attn_backend.get_kv_cache_stride_order(include_num_layers_dimension=True))
        except (AttributeError, NotImplementedError, TypeError):
            order = tuple(range(kv_cache.dim()))
        if sorted(order) != list(range(kv_cache.dim())):
            raise ValueError(f"stride order {order} does not match a {kv_cache.dim()}-D KV tensor")
        logical = kv_cache.permute(*[order.index(i) for i in range(len(order))])  # (layers, per-layer shape)
        self.register_kv_caches({f"layer.{i}": logical[i] for i in range(logical.shape[0])})

    def register_kv_caches(self, kv_caches: dict[str, torch.Tensor]) -> None:
        info = describe_kv_caches(kv_caches)
        first = kv_caches[info["names"][0]]
        # each tensor-parallel worker stores its own head slice in its own file
        geo = KVGeometry(len(info["names"]), info["heads"], info["head_dim"], info["block_tokens"],
                         first.element_size(), self._codec)
        if self._slot_size and self._tp == 1 and geo.slot_size != self._slot_size:
            raise ValueError(f"configured slot_size {self._slot_size} != derived {geo.slot_size}")
        store_path = self._store_path if self._tp == 1 else f"{self._store_path}.tp{self._rank}"
        self._layer_names = info["names"]
        st = info["strides"]
        if first.is_cuda:
            from daser_b200.kv.hbm_store import HBMStore
            from daser_b200.ops import kv_ops

            if first.dtype != torch.bfloat16:
                raise ValueError("the CUDA connector path expects a bf16 KV cache")
            pool = kv_ops.PagedKVPool(
                payload_ptrs=[first.data_ptr()], scale_ptrs=[0], stride_layer=info["layer_stride"],
                stride_block=st["N"], stride_kv=st["K"], stride_tok=st["T"], stride_head=st["H"],
                num_blocks=info["num_blocks"], heads_per_rank=info["heads"], is_fp8=False,
                keepalive=[kv_caches],
            )
            inv_freq = [1.0] * (info["head_dim"] // 2)  # prefix reuse never rotates (delta = 0)
            backend: Any = CudaKVBackend(geo, pool, inv_freq, max_pos=2)
            hbm = HBMStore(geo.slot_size, self._hbm_slots) if self._hbm_slots else None
            host = HBMStore(geo.slot_size, self._host_slots, torch.device("cpu")) if self._host_slots else None
        else:
            stacked = torch.stack([kv_caches[n] for n in info["names"]])  # CPU test path: a copy
            order = "L" + info["layout"]
            view = stacked.permute([order.index(c) for c in "LNKHTD"])
            backend = _CpuViewBackend(geo, view, kv_caches, info)
            hbm = host = None
        self._worker = WorkerHalf(self._socket_path, store_path, geo, backend, io_backend=self._io_backend,
                                  tp=1, rank=0, hbm_store=hbm, host_store=host,
                                  staging_slots=self._staging_slots, write_behind=self._write_behind)
        if self._tp > 1:
            self._worker.commit_parts = (self._rank, self._tp)
        logger.info("[CONNECTOR] registered %d KV layers, layout %s, slot_size=%d, backend=%s",
                    len(info["names"]), info["layout"], geo.slot_size, self._worker.transfer.backend.name)

    def bind_connector_metadata(self, connector_metadata: Any) -> None:
        super().bind_connector_metadata(connector_metadata)
        if self._worker is not None:
            self._worker.bind_connector_metadata(
                ConnectorMeta(list(connector_metadata.reqs_to_load), list(connector_metadata.reqs_to_store)))

    def clear_connector_metadata(self) -> None:
        super().clear_connector_metadata()
        if self._worker is not None:
            self._worker.clear_connector_metadata()

    def start_load_kv(self, forward_context: Any = None, **kwargs: Any) -> None:
        if self._worker is not None:
            self._worker.start_load_kv()

    @classmethod
    def requires_piecewise_for_cudagraph(cls, extra_config: dict[str, Any]) -> bool:
        """No: nothing happens in the per-layer hooks (restore completes in :meth:`start_load_kv`,
        save gathers all layers in :meth:`wait_for_save`), so a full-graph replay that skips them
        loses nothing.  The reference had to make its loads synchronous for the same reason
        (``docs/design/architecture.md:48-52`` there)."""
        return False

    def wait_for_layer_load(self, layer_name: str) -> None:
        """Loads finish inside :meth:`start_load_kv`; a full CUDA-graph replay skips Python hooks."""

    def save_kv_layer(self, layer_name: str, kv_layer: Any = None, attn_metadata: Any = None, **kwargs: Any) -> None:
        """Nothing per layer: all layers are gathered by one launch in :meth:`wait_for_save`."""

    def wait_for_save(self) -> None:
        if self._worker is not None:
            self._worker.wait_for_save()

    def get_block_ids_with_load_errors(self) -> set[int]:
        return self._worker.take_load_errors() if self._worker is not None else set()

    def reset_cache(self) -> bool:
        """Drop what this connector caches itself (the HBM and pinned-host tiers).  The store file
        and the control plane's index are shared with other engines and are left alone."""
        if self._worker is not None:
            for tier in (self._worker.hbm, self._worker.host):
                if tier is not None:
                    tier.clear()
        return True

    def get_kv_connector_stats(self) -> Any:
        """What this worker moved since the last call, in vLLM's stats container (None when
        nothing happened, or when the installed vLLM has no such container)."""
        if self._worker is None or DaserKVConnectorStats is None:
            return None
        now = self._worker.get_stats()
        delta = {k: now.get(k, 0) - self._stats_seen.get(k, 0) for k in _STAT_KEYS}
        self._stats_seen = {k: now.get(k, 0) for k in _STAT_KEYS}
        if not any(delta.values()):
            return None
        return DaserKVConnectorStats(data={k.split(".", 1)[1]: v for k, v in delta.items()})

    @classmethod
    def build_kv_connector_stats(cls, data: Optional[dict[str, Any]] = None) -> Any:
        if DaserKVConnectorStats is None:
            return None
        return DaserKVConnectorStats(data=dict(data)) if data is not None else DaserKVConnectorStats()

    @classmethod
    def build_prom_metrics(cls, vllm_config: Any, metric_types: Any, labelnames: list[str],
                           per_engine_labelvalues: dict[int, list[object]]) -> Any:
        """vLLM's logger process calls this once and then feeds it every reduced stats interval."""
        if DaserPromMetrics is None:
            return None
        return DaserPromMetrics(vllm_config, metric_types, labelnames, per_engine_labelvalues)

    def get_stats(self) -> dict[str, float]:
        return self._worker.get_stats() if self._worker is not None else {}

    def shutdown(self) -> None:
        if self._worker is not None:
            self._worker.shutdown()
            self._worker = None
        if self._sched is not None:
            self._sched.close()
            self._sched = None


class _CpuViewBackend(TorchKVBackend):
    """CPU KV tensors in vLLM's own layout: restore/save through a stacked copy that is
    written back to (read from) the engine's per-layer tensors."""

    def __init__(self, geo: KVGeometry, view: torch.Tensor, kv_caches: dict[str, torch.Tensor], info: dict) -> None:
        super().__init__(geo, view.contiguous(), [1.0] * (geo.head_dim // 2))
        self._caches, self._info = kv_caches, info

    def _to_engine(self) -> None:
        order = "L" + self._info["layout"]
        back = self.pool.permute(["LNKHTD".index(c) for c in order])
        for i, name in enumerate(self._info["names"]):
            self._caches[name].copy_(back[i])

    def _from_engine(self) -> None:
        order = "L" + self._info["layout"]
        stacked = torch.stack([self._caches[n] for n in self._info["names"]])
        self.pool.copy_(stacked.permute([order.index(c) for c in "LNKHTD"]))

    def restore(self, images, block_ids, deltas) -> None:
        self._from_engine()
        super().restore(images, block_ids, deltas)
        self._to_engine()

    def save(self, block_ids, images) -> None:
        self._from_engine()
        super().save(block_ids, images)
