"""Tensor parallelism over NVLink peer memory: symmetric buffers, counters, fused forward.

The reference has no tensor parallelism (its connector is not rank aware: every rank would
write the same file offsets, ``daser/connector/daser_connector.py:150-156,652``); the stack it
is benchmarked with (stock vLLM) runs row-parallel GEMMs followed by a separate NCCL /
custom all-reduce (``vllm/model_executor/layers/linear.py``).  Here one process drives one
GPU and the hot path makes no NCCL call:

* **GEMM -> reduce-scatter** is the epilogue of the tcgen05 GEMM (``ops/csrc/gemm.cu``): every
  partial tile leaves TMEM straight into the fp32 accumulator of the rank that owns those
  rows (vector ``red.global.add`` on peer-mapped memory), then bumps that rank's arrival
  counter.
* **all-gather -> GEMM**: the add + RMSNorm kernel of the row owner waits for the arrivals,
  normalises its rows and stores them into every rank's gathered-activation buffer (plain
  16-byte peer stores), then bumps a per-source flag on every rank; the TMA producer of the
  next column-parallel GEMM waits for exactly the flags of the rows its tile needs.
* **steps of few tokens at tp <= 2** use the one-shot form instead: the GEMM epilogue writes its
  partial into every peer's receive buffer and each rank sums and normalises all rows itself: one
  NVLink hop per sync point, no all-gather (``_forward_body_oneshot``).  At higher degrees the
  tp - 1 copies cost more than the second hop saves (measured), so the two-hop form stays.
* **in-switch form** (``impl="nvls"``, opt-in): the GEMM keeps its partial in its own memory and only
  signals; each rank's add + RMSNorm reads the sum of all ranks' partials through the NVLink
  multicast mapping (``multimem.ld_reduce``: the switch adds in flight).  One hop, T x hidden x 2
  bytes in per rank whatever tp is.  Needs multicast-mapped buffers (below).
* **chunk-KV restore** scatters from the IO rank into every rank's paged pool
  (``ops/csrc/kv_paged.cu``); **save** has every rank compress and push its head slice into
  the IO rank's staging buffer.

NCCL is used for bootstrap, barriers between engine steps and the gathered logits rows of
top-k / top-p requests; the sampling candidates (8 bytes per sequence and rank) are exchanged by
``tp_pick_token_kernel`` over peer memory.  Only the opt-in in-switch form uses ``multimem``, so by
default the symmetric allocations are made without an NVLink multicast object bound to them
(``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` unless the caller set it, or asked for ``multicast``): a
process that dies while its memory is bound to one raises NVLink faults on its peers' GPUs.  Peer liveness is checked on the
host between steps (:mod:`daser_b200.parallel.health`).  Buffers that peers touch are allocated with
``torch.distributed._symmetric_memory`` (VMM allocations exchanged between the processes).
All device-side waits are bounded and report through a status word.
"""

from __future__ import annotations

import os
from typing import Any, Optional

import torch
import torch.distributed as dist

from daser_b200.models.llama import LlamaConfig
from daser_b200.ops import attention, elementwise as ew, gemm, kv_ops
from daser_b200.parallel.health import PeerMonitor
from daser_b200.parallel.mailbox import open_mailbox

FLAG_RS = 0  # arrival counter of reduce-scattered partials
FLAG_OS = 1  # and 2: arrival counters of the two one-shot all-reduce receive buffers
# Largest degree at which "fused" picks the one-shot form for small steps.  Measured on the 70B
# 64-token step (compute part, ms): tp = 2: one-shot 21.7, two-hop 22.4, NCCL 21.7; tp = 8: one-shot
# 19.9, two-hop 14.3, NCCL 15.2.  The one-shot epilogue sends tp - 1 copies of every tile; at 8
# ranks those stores dominate the GEMM's epilogue.
ONESHOT_MAX_TP = 2
FLAG_NV = 3  # and 4: arrival counters of the two in-switch all-reduce buffers
FLAG_CAND = 5  # arrival counter of the sampling candidates
FLAG_AG = 8  # first of tp per-source "rows landed" flags
FLAG_KV = 16  # first of tp per-source "restore pieces landed in your pool" counters
NUM_FLAGS = 24
IMPLS = ("fused", "twoshot", "oneshot", "nvls", "nccl")


class TPContext:
    def __init__(self, cfg: LlamaConfig, group: Any, max_tokens: int = 256, impl: Optional[str] = None,
                 multicast: Optional[bool] = None) -> None:
        # "fused": the path this module is about.  "nccl": the unfused arrangement it is measured
        # against (same kernels, replicated activations, NCCL all-reduce after the row-parallel GEMMs).
        # "twoshot" / "oneshot" force one form of the fused reduction at every size and degree.
        # "nvls": the in-switch form (needs `multicast`); opt-in, see `_forward_body_nvls`.
        self.impl = impl or os.environ.get("DASER_TP_IMPL", "fused")
        if self.impl not in IMPLS:
            raise ValueError(f"unknown tensor-parallel implementation {self.impl!r}")
        # Symmetric allocations get an NVLink multicast mapping only on request: a process that dies
        # while its memory is bound to one raises NVLink faults on its peers' GPUs, so deployments
        # that must survive a lost rank keep it off.
        if multicast is None:
            multicast = self.impl == "nvls" or os.environ.get("DASER_TP_MULTICAST", "0") == "1"
        self.multicast = bool(multicast)
        if self.multicast:
            if os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST") == "1":
                raise ValueError("multicast requested but TORCH_SYMM_MEM_DISABLE_MULTICAST=1 is set")
        else:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.cfg = cfg
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.group_name = group.group_name
        self._cpu_group = dist.new_group(backend="gloo")
        self._tensors: dict[str, torch.Tensor] = {}
        self._handles: dict[str, Any] = {}
        self.ptrs: dict[str, list[int]] = {}
        self.max_tokens = max_tokens
        self.rows_max = -(-max_tokens // self.tp)
        H = cfg.hidden
        # peers reduce into `acc`, push into `gathered`, and bump `flags`
        self.acc = self.alloc("acc", (self.tp * self.rows_max, H), torch.bfloat16)  # [source rank][row][H]
        self.gathered = self.alloc("gathered", (self.rows_max * self.tp, H), torch.bfloat16)
        self.flags = self.alloc("flags", (NUM_FLAGS,), torch.int32)
        self.acc.zero_()
        self.gathered.zero_()
        self.flags.zero_()
        # local only
        self.h_local = torch.zeros(self.rows_max, H, dtype=torch.bfloat16, device=self.device)
        self.done = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.tile_counters = torch.zeros(4096, dtype=torch.int32, device=self.device)
        # sampling: every rank's best (value, index) per row lands in every rank's table
        # ([2 rounds][tp sources][value, index][CAND_CAP rows]); `epoch_cand` counts consumed arrivals
        self.cand_cap = 64
        self.cand = self.alloc("cand", (2 * self.tp * 2 * self.cand_cap,), torch.float32)
        self.cand.zero_()
        self.epoch_cand = torch.zeros(1, dtype=torch.int32, device=self.device)
        # device-resident bases of the three growing counters (reduce-scatter arrivals, pushes
        # per source rank, finished norm CTAs): kernels wait for base + offset, and the last
        # kernel of a forward advances the bases, so a captured forward can be replayed
        self.epochs = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._rs_off = self._ag_off = self._done_off = 0
        # one-shot all-reduce (steps of few tokens): two alternating receive buffers of tp slots
        # x os_cap rows, their arrival counters and the bases those counters are read against
        self.os_cap = min(max_tokens, int(os.environ.get("DASER_TP_ONESHOT_MAX", "256")))
        self.os_buf = [self.alloc(f"os_{i}", (self.tp * self.os_cap, H), torch.bfloat16) for i in range(2)]
        self.epochs_os = torch.zeros(4, dtype=torch.int32, device=self.device)
        # in-switch all-reduce: two alternating buffers that hold this rank's own partial (os_cap rows);
        # peers read the sum of all ranks' buffers through the multicast alias of the same range
        self.nv_buf: list[torch.Tensor] = []
        self.nv_mc: list[int] = []
        # steps of up to this many tokens take the in-switch form (its add + norm kernel handles one
        # wave of rows: one CTA per row, 148 SMs); longer ones take the two-hop form
        self.nv_cap = min(self.os_cap, int(os.environ.get("DASER_TP_NVLS_MAX", "128")))
        self.epochs_nv = torch.zeros(4, dtype=torch.int32, device=self.device)
        if self.multicast:
            for i in range(2):
                self.nv_buf.append(self.alloc(f"nv_{i}", (self.os_cap, H), torch.bfloat16))
                self.nv_buf[i].zero_()
                self.nv_mc.append(int(getattr(self._handles[f"nv_{i}"], "multicast_ptr", 0) or 0))
            if not all(self.nv_mc):
                if self.impl == "nvls":
                    raise RuntimeError("no NVLink multicast mapping for the symmetric buffers (NVLS unavailable)")
                self.nv_buf, self.nv_mc = [], []
        self.save_staging: Optional[torch.Tensor] = None
        self._mail_timeout = float(os.environ.get("DASER_TP_MAIL_TIMEOUT", "120"))
        self.mailbox = None
        self.health: Optional[PeerMonitor] = None
        if os.environ.get("DASER_TP_HEALTH", "1") != "0":
            store = dist.distributed_c10d._get_default_store()
            self.health = PeerMonitor(dist.PrefixStore(f"daser/{self.group_name}", store), self.rank, self.tp,
                                      timeout_s=float(os.environ.get("DASER_TP_HEALTH_TIMEOUT", "10")))
        # per-step control messages (plans, load-error reports) go through shared memory, not gloo
        self.mailbox = open_mailbox(self.rank, self.tp, self._broadcast_gloo)
        torch.cuda.synchronize()
        self.barrier()

    # -- plumbing -------------------------------------------------------------------------
    def alloc(self, name: str, shape, dtype) -> torch.Tensor:
        """A tensor every rank can address: returns the local one, records all ranks' pointers."""
        t = self._symm.empty(tuple(shape), dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self.group_name)
        self._tensors[name], self._handles[name] = t, hdl
        self.ptrs[name] = [int(p) for p in hdl.buffer_ptrs]
        return t

    def barrier(self) -> None:
        dist.barrier(group=self.group, device_ids=[self.device.index])

    def check_peers(self) -> None:
        """Raise :class:`~daser_b200.parallel.health.PeerLost` if a peer left or stopped beating.

        Called between engine steps, before anything that waits on a peer is launched."""
        if self.health is not None:
            self.health.check()

    def multicast_bound(self) -> bool:
        """True if any symmetric allocation of this context has an NVLink multicast mapping."""
        return any(int(getattr(h, "multicast_ptr", 0) or 0) != 0 for h in self._handles.values())

    def leave(self) -> None:
        """Orderly exit of this rank: between steps, after its own work has drained."""
        torch.cuda.synchronize()
        if self.health is not None:
            self.health.leave()

    def close(self) -> None:
        if self.health is not None:
            self.health.close()
        if self.mailbox is not None:
            self.mailbox.close()
            self.mailbox = None

    def _broadcast_gloo(self, obj: Any, src: int = 0) -> Any:
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self._cpu_group)
        return box[0]

    def broadcast_object(self, obj: Any, src: int = 0, timeout_s: Optional[float] = None) -> Any:
        """``obj`` of rank ``src`` on every rank.  Through the shared-memory mailbox (microseconds);
        a peer that stops publishing surfaces as :class:`~daser_b200.parallel.health.PeerLost` or a
        time-out instead of a hung collective.  ``timeout_s=float("inf")`` waits as long as the
        peers stay alive (a follower of an idle service waiting for the leader's next call)."""
        if self.mailbox is None:
            return self._broadcast_gloo(obj, src)
        return self.mailbox.broadcast(obj, src, timeout_s=self._mail_timeout if timeout_s is None else timeout_s,
                                      on_wait=self.check_peers)

    def await_announcement(self, obj: Any = None, src: int = 0) -> Any:
        """:meth:`broadcast_object` without a time limit: what a follower waits for between requests."""
        return self.broadcast_object(obj, src, timeout_s=float("inf"))

    def gather_object(self, obj: Any) -> list:
        """Every rank's ``obj`` in rank order, on every rank."""
        if self.mailbox is None:
            out: list = [None] * self.tp
            dist.all_gather_object(out, obj, group=self._cpu_group)
            return out
        return self.mailbox.gather(obj, timeout_s=self._mail_timeout, on_wait=self.check_peers)

    def wait_for_path(self, path: str, timeout_s: float = 60.0) -> None:
        """Block until ``path`` exists (a file another rank creates)."""
        import time

        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"{path} did not appear")
            time.sleep(0.01)

    # -- restore hand-shake: "my scatter into your pool has landed" -------------------------------
    def signal_kv_landed(self, value: int) -> None:
        """On the current stream, behind this rank's restore kernel: publish ``value`` (a count of
        finished restore pieces that only grows) in this rank's slot of every rank's counters."""
        ew.signal_flags([self.flag_ptr(r, FLAG_KV + self.rank) for r in range(self.tp)], value)

    def wait_kv_landed(self, value: int, status: Optional[torch.Tensor]) -> None:
        """On the current stream: a bounded wait until every rank's counter here has reached ``value``."""
        ew.wait_flags(self.flag_ptr(self.rank, FLAG_KV), self.tp, value, status)

    def global_pool(self, runner) -> kv_ops.PagedKVPool:
        """The paged pool as the restore / save kernels see it: one base pointer per rank."""
        local = runner.local_pool
        return kv_ops.PagedKVPool(
            payload_ptrs=self.ptrs["kv_payload"], scale_ptrs=self.ptrs["kv_scales"],
            stride_layer=local.stride_layer, stride_block=local.stride_block, stride_kv=local.stride_kv,
            stride_tok=local.stride_tok, stride_head=local.stride_head, num_blocks=local.num_blocks,
            heads_per_rank=local.heads_per_rank, is_fp8=True, keepalive=[runner.kv_payload, runner.kv_scales],
        )

    def flag_ptr(self, rank: int, index: int) -> int:
        return self.ptrs["flags"][rank] + 4 * index

    # -- fused building blocks ---------------------------------------------------------------
    def _norm_push(self, runner, x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor],
                   rows: int, wait: bool) -> None:
        """Add + RMSNorm on this rank's ``rows`` rows, pushed into every rank's ``gathered``."""
        sync = ew.TpSync()
        ep = self.epochs.data_ptr()
        if wait:
            sync.wait_counter = self.flag_ptr(self.rank, FLAG_RS)
            sync.wait_target = self._rs_off
            sync.wait_base = ep
        self._done_off += rows
        sync.done_counter = self.done.data_ptr()
        sync.done_target = self._done_off
        sync.done_base = ep + 8
        for r in range(self.tp):
            sync.signal[r] = self.flag_ptr(r, FLAG_AG + self.rank)
        sync.n_signal = self.tp
        sync.status = runner.status.data_ptr()
        self._ag_off += 1
        # after a reduce-scatter, x is the receive buffer: tp slots of `rows` partial rows each
        ew.add_rmsnorm(x[:rows], weight, residual=residual, eps=self.cfg.rms_eps, zero_after=False,
                       out_ptrs=self.ptrs["gathered"], out_row_offset=self.rank * rows, tp_sync=sync,
                       n_partials=self.tp if wait else 1, partial_stride=rows * self.cfg.hidden)

    def _col_gemm(self, runner, w: torch.Tensor, acc: torch.Tensor, out_bf: torch.Tensor, T: int, rows: int):
        """all-gather -> GEMM: A is the gathered activation, loads gated on the per-source flags."""
        x = self.gathered[:T]
        bn, ks = gemm.plan_tiles(T, w.shape[0], w.shape[1], allow_split=True)
        gate = dict(gate_flags=self.flag_ptr(self.rank, FLAG_AG), gate_target=self._ag_off, gate_rows=rows,
                    gate_base=self.epochs.data_ptr() + 4)
        if ks > 1:
            gemm.linear(x, w, acc=acc[:T], block_n=bn, k_splits=ks, status=runner.status, **gate)
            return acc[:T], True
        gemm.linear(x, w, out=out_bf[:T], block_n=bn, k_splits=1, status=runner.status, **gate)
        return out_bf[:T], False

    def _row_gemm(self, runner, x: torch.Tensor, w: torch.Tensor, T: int, rows: int) -> None:
        """GEMM -> reduce-scatter: every partial tile is stored (bf16) into this rank's slot of
        the row owner's receive buffer; the owner's norm kernel sums the slots."""
        N, K = w.shape
        # measured (M = 64, N = 8192): plain bf16 stores from 64-wide tiles win up to K ~ 4k per rank,
        # split-K with the last-CTA scatter wins beyond
        bn, ks = (128, 4) if K >= 8192 and T <= 128 else (64, 1)
        if -(-T // 128) * -(-N // 128) >= 148:
            bn, ks = 128, 1
        counts = gemm.expected_arrivals(T, N, bn, 1, rows, self.tp, K)  # one arrival per tile, whatever ks
        self._rs_off += self.tp * counts[self.rank]
        gemm.linear(x, w, owners=self.ptrs["acc"], rows_per_owner=rows, ldc=N, block_n=bn, k_splits=ks,
                    scatter_bf16=True, dst_row_offset=self.rank * rows, work=runner.hid_acc[:T],
                    tile_counters=self.tile_counters,
                    arrive=[self.flag_ptr(r, FLAG_RS) for r in range(self.tp)], status=runner.status)

    # -- the model step ---------------------------------------------------------------------------
    @torch.no_grad()
    def forward_body(self, runner, inp, nsplit: int, split_tokens: int, l0: int = 0, l1: Optional[int] = None) -> None:
        """Layers ``[l0, l1)`` (the embedding in front of layer 0, the final norm push behind the last
        layer); ends by advancing the epoch bases, so consecutive layer ranges chain: the first
        wait of a range finds the previous range's last pushes at offset 0 of the new bases.

        Every launch depends only on the step's shape (offsets are relative to the bases), so
        the runner may capture this body in a CUDA graph and replay it.  Counter comparisons
        are wrap-safe (signed difference), so the 32-bit counters may grow for ever.
        """
        cfg, w = self.cfg, runner.w
        T = inp.num_tokens
        if T > self.max_tokens or T > runner.max_tokens:
            raise ValueError("step exceeds the tensor-parallel buffers")
        l1 = len(w.layers) if l1 is None else l1
        if self.impl == "nccl":
            return self._forward_body_nccl(runner, inp, nsplit, split_tokens, l0, l1)
        if self.impl == "nvls" and T <= self.nv_cap:
            # (longer steps, the prefill pieces, take the two-hop form below: its buffers hold max_tokens)
            return self._forward_body_nvls(runner, inp, nsplit, split_tokens, l0, l1)
        if self.impl == "oneshot" or (self.impl == "fused" and self.tp <= ONESHOT_MAX_TP and T <= self.os_cap):
            return self._forward_body_oneshot(runner, inp, nsplit, split_tokens, l0, l1)
        self._rs_off = self._ag_off = self._done_off = 0
        D, B = cfg.head_dim, cfg.block_tokens
        rows = -(-T // self.tp)
        first = self.rank * rows
        mine = max(0, min(rows, T - first))
        h = self.h_local[:rows]
        if l0 == 0:
            if mine < rows:
                h[mine:].zero_()
            if mine > 0:
                ew.embedding(inp.tokens[first : first + mine], w.embed, out=h[:mine])
            self._norm_push(runner, h, w.layers[0].input_norm, None, rows, wait=False)
        for li in range(l0, l1):
            lw = w.layers[li]
            # all-gather -> QKV GEMM (loads gated on the per-source flags) -> RoPE + KV write in its epilogue
            runner.qkv_rope(self.gathered[:T], lw, inp, T, li, gate_flags=self.flag_ptr(self.rank, FLAG_AG),
                            gate_target=self._ag_off, gate_rows=rows, gate_base=self.epochs.data_ptr() + 4)
            attn = runner.attn_out[:T].view(T, runner.hq, D)
            attention.paged_attention(runner.q_rot[:T], attn, runner.local_pool, li, inp.block_tables, inp.q_start,
                                      inp.ctx_lens, inp.max_q_len, inp.max_ctx, runner.hkv, runner.softmax_scale,
                                      runner.attn_ws, nsplit=nsplit, split_tokens=split_tokens)
            self._row_gemm(runner, runner.attn_out[:T], lw.wo, T, rows)
            self._norm_push(runner, self.acc, lw.post_norm, h, rows, wait=True)
            runner.mlp_up(self.gathered[:T], lw, T, gate_flags=self.flag_ptr(self.rank, FLAG_AG),
                          gate_target=self._ag_off, gate_rows=rows, gate_base=self.epochs.data_ptr() + 4)
            self._row_gemm(runner, runner.act[:T], lw.w_down, T, rows)
            nxt = w.layers[li + 1].input_norm if li + 1 < len(w.layers) else w.final_norm
            self._norm_push(runner, self.acc, nxt, h, rows, wait=True)
        ew.advance_epochs(self.epochs, self._rs_off, self._ag_off, self._done_off)

    # -- one-shot form: GEMM -> all-reduce in the epilogue, one NVLink hop per sync point -----------
    def _row_gemm_bcast(self, runner, x: torch.Tensor, w: torch.Tensor, T: int, which: int, offs: list[int]) -> None:
        """Row-parallel GEMM whose epilogue stores the bf16 partial into this rank's slot of EVERY
        rank's receive buffer ``which`` and bumps every rank's arrival counter once per tile."""
        N, K = w.shape
        bn, ks = (128, 4) if K >= 8192 and T <= 128 else (64, 1)
        if -(-T // 128) * -(-N // 128) >= 148:
            bn, ks = 128, 1
        offs[which] += self.tp * -(-T // 128) * -(-N // bn)
        gemm.linear(x, w, owners=self.ptrs[f"os_{which}"], rows_per_owner=self.os_cap, ldc=N, block_n=bn,
                    k_splits=ks, scatter_bf16=True, dst_row_offset=self.rank * self.os_cap, broadcast=True,
                    work=runner.hid_acc[:T], tile_counters=self.tile_counters,
                    arrive=[self.flag_ptr(r, FLAG_OS + which) for r in range(self.tp)], status=runner.status)

    def _norm_sum(self, runner, which: int, weight: torch.Tensor, h: torch.Tensor, out: torch.Tensor, T: int,
                  offs: list[int]) -> None:
        """Wait for every rank's partial in buffer ``which``, sum the tp slots, add the residual and
        normalise all T rows locally (every rank sums the same values in the same order, so the
        replicated residual streams stay bit-identical)."""
        sync = ew.TpSync()
        sync.wait_counter = self.flag_ptr(self.rank, FLAG_OS + which)
        sync.wait_target = offs[which]
        sync.wait_base = self.epochs_os.data_ptr() + 4 * which
        sync.status = runner.status.data_ptr()
        ew.add_rmsnorm(self.os_buf[which][:T], weight, residual=h, out=out, eps=self.cfg.rms_eps, zero_after=False,
                       tp_sync=sync, n_partials=self.tp, partial_stride=self.os_cap * self.cfg.hidden)

    def _forward_body_oneshot(self, runner, inp, nsplit: int, split_tokens: int, l0: int, l1: int) -> None:
        """The fused forward for steps of few tokens (a RAG query block, a decode batch).

        At this size a sync point costs latency, not bandwidth, so each of the two per-layer
        reductions is ONE hop: the row-parallel GEMM's epilogue writes its bf16 partial tile
        straight into every peer's receive buffer while the other tiles still compute, and each
        rank's add + RMSNorm waits for the arrivals, sums the tp slots from its own HBM and
        normalises all rows; the next column-parallel GEMM then reads local memory and needs no
        gate.  The price is tp - 1 times the reduce-scatter's NVLink bytes (7 MB per GEMM at 64
        tokens and tp = 8), spread over the GEMM.  The two receive buffers alternate: a peer can
        only overwrite a buffer after it has passed the other one's sync point, which needs this
        rank's next partial, which this rank issues after it has read the first."""
        cfg, w = self.cfg, runner.w
        T = inp.num_tokens
        D, B = cfg.head_dim, cfg.block_tokens
        h, normed = runner.h[:T], runner.normed[:T]
        offs = [0, 0]
        if l0 == 0:
            ew.embedding(inp.tokens, w.embed, out=h)
            ew.add_rmsnorm(h, w.layers[0].input_norm, out=normed, eps=cfg.rms_eps)
        for li in range(l0, l1):
            lw = w.layers[li]
            runner.qkv_rope(normed, lw, inp, T, li)
            attn = runner.attn_out[:T].view(T, runner.hq, D)
            attention.paged_attention(runner.q_rot[:T], attn, runner.local_pool, li, inp.block_tables, inp.q_start,
                                      inp.ctx_lens, inp.max_q_len, inp.max_ctx, runner.hkv, runner.softmax_scale,
                                      runner.attn_ws, nsplit=nsplit, split_tokens=split_tokens)
            self._row_gemm_bcast(runner, runner.attn_out[:T], lw.wo, T, 0, offs)
            self._norm_sum(runner, 0, lw.post_norm, h, normed, T, offs)
            runner.mlp_up(normed, lw, T)
            self._row_gemm_bcast(runner, runner.act[:T], lw.w_down, T, 1, offs)
            last = li + 1 == len(w.layers)
            nxt = w.final_norm if last else w.layers[li + 1].input_norm
            self._norm_sum(runner, 1, nxt, h, self.gathered[:T] if last else normed, T, offs)
        ew.advance_epochs(self.epochs_os, offs[0], offs[1], 0)

    # -- in-switch form: partial stays local, the reader sums through the NVLink multicast mapping ----
    def _forward_body_nvls(self, runner, inp, nsplit: int, split_tokens: int, l0: int, l1: int) -> None:
        """The one-shot form with the NVSwitch doing the sum.

        Each row-parallel GEMM stores its bf16 partial into this rank's OWN buffer (local stores
        only: nothing crosses NVLink in the epilogue) and bumps every rank's arrival counter; each
        rank's add + RMSNorm waits for the tp x tiles arrivals and then reads every row through
        the multicast alias with ``multimem.ld_reduce`` (the switch fetches the tp partials and adds
        them in fp32 on the way), adds the residual and normalises all rows.  Per sync point and
        rank: T x hidden x 2 bytes come in over NVLink, whatever tp is, against tp - 1 times that
        going out in the store form; one hop, no all-gather, two sync points per layer.  Buffer
        reuse follows the one-shot form's argument (two alternating buffers; a rank can only pass
        sync point k + 1 after every peer has finished reading at sync point k).

        Needs symmetric buffers with a multicast mapping (``multicast=True``), which a deployment
        that must survive a lost rank keeps off: hence opt-in.
        """
        if not self.nv_mc:
            raise RuntimeError("the in-switch form needs a context built with multicast=True")
        cfg, w = self.cfg, runner.w
        T = inp.num_tokens
        if T > self.nv_cap:
            raise ValueError("step exceeds the in-switch all-reduce buffers")
        D, B = cfg.head_dim, cfg.block_tokens
        h, normed = runner.h[:T], runner.normed[:T]
        offs = [0, 0]

        def row_gemm(x: torch.Tensor, wt: torch.Tensor, which: int) -> None:
            N, K = wt.shape
            bn, ks = (128, 4) if K >= 8192 and T <= 128 else (64, 1)
            if -(-T // 128) * -(-N // 128) >= 148:
                bn, ks = 128, 1
            offs[which] += self.tp * -(-T // 128) * -(-N // bn)
            gemm.linear(x, wt, owners=[self.nv_buf[which].data_ptr()] * self.tp, rows_per_owner=self.os_cap, ldc=N,
                        block_n=bn, k_splits=ks, scatter_bf16=True, dst_row_offset=0, signal_all=True,
                        work=runner.hid_acc[:T], tile_counters=self.tile_counters,
                        arrive=[self.flag_ptr(r, FLAG_NV + which) for r in range(self.tp)], status=runner.status)

        def norm_sum(which: int, weight: torch.Tensor, out: torch.Tensor) -> None:
            sync = ew.TpSync()
            sync.wait_counter = self.flag_ptr(self.rank, FLAG_NV + which)
            sync.wait_target = offs[which]
            sync.wait_base = self.epochs_nv.data_ptr() + 4 * which
            sync.status = runner.status.data_ptr()
            sync.mc_x = self.nv_mc[which]
            ew.add_rmsnorm(self.nv_buf[which][:T], weight, residual=h, out=out, eps=cfg.rms_eps, zero_after=False,
                           tp_sync=sync)

        if l0 == 0:
            ew.embedding(inp.tokens, w.embed, out=h)
            ew.add_rmsnorm(h, w.layers[0].input_norm, out=normed, eps=cfg.rms_eps)
        for li in range(l0, l1):
            lw = w.layers[li]
            runner.qkv_rope(normed, lw, inp, T, li)
            attn = runner.attn_out[:T].view(T, runner.hq, D)
            attention.paged_attention(runner.q_rot[:T], attn, runner.local_pool, li, inp.block_tables, inp.q_start,
                                      inp.ctx_lens, inp.max_q_len, inp.max_ctx, runner.hkv, runner.softmax_scale,
                                      runner.attn_ws, nsplit=nsplit, split_tokens=split_tokens)
            row_gemm(runner.attn_out[:T], lw.wo, 0)
            norm_sum(0, lw.post_norm, normed)
            runner.mlp_up(normed, lw, T)
            row_gemm(runner.act[:T], lw.w_down, 1)
            last = li + 1 == len(w.layers)
            norm_sum(1, w.final_norm if last else w.layers[li + 1].input_norm, self.gathered[:T] if last else normed)
        ew.advance_epochs(self.epochs_nv, offs[0], offs[1], 0)

    def _forward_body_nccl(self, runner, inp, nsplit: int, split_tokens: int, l0: int, l1: int) -> None:
        """The baseline: what stock tensor parallelism does (``vllm/model_executor/layers/linear.py``,
        ``RowParallelLinear`` with ``reduce_results``): every rank keeps the whole residual stream,
        column- and row-parallel GEMMs run on the local shards (the same tcgen05 kernels as the
        fused path), and the row-parallel outputs are summed by a NCCL all-reduce (on the fp32
        split-K accumulator when the GEMM was split, else on its bf16 output) before the
        add + RMSNorm, which every rank repeats on all rows.  No peer memory, no flags."""
        cfg, w = self.cfg, runner.w
        T = inp.num_tokens
        D, B = cfg.head_dim, cfg.block_tokens
        h, normed = runner.h[:T], runner.normed[:T]
        if l0 == 0:
            ew.embedding(inp.tokens, w.embed, out=h)
            ew.add_rmsnorm(h, w.layers[0].input_norm, out=normed, eps=cfg.rms_eps)
        for li in range(l0, l1):
            lw = w.layers[li]
            runner.qkv_rope(normed, lw, inp, T, li)
            attn = runner.attn_out[:T].view(T, runner.hq, D)
            attention.paged_attention(runner.q_rot[:T], attn, runner.local_pool, li, inp.block_tables, inp.q_start,
                                      inp.ctx_lens, inp.max_q_len, inp.max_ctx, runner.hkv, runner.softmax_scale,
                                      runner.attn_ws, nsplit=nsplit, split_tokens=split_tokens)
            o, f32 = runner._linear(runner.attn_out[:T], lw.wo, runner.hid_acc, runner.hid_bf)
            dist.all_reduce(o, group=self.group)
            ew.add_rmsnorm(o, lw.post_norm, residual=h, out=normed, eps=cfg.rms_eps, zero_after=f32)
            runner.mlp_up(normed, lw, T)
            d, f32 = runner._linear(runner.act[:T], lw.w_down, runner.hid_acc, runner.hid_bf)
            dist.all_reduce(d, group=self.group)
            nxt = w.layers[li + 1].input_norm if li + 1 < len(w.layers) else w.final_norm
            ew.add_rmsnorm(d, nxt, residual=h, out=normed, eps=cfg.rms_eps, zero_after=f32)
        if l1 == len(w.layers):
            self.gathered[:T].copy_(normed)  # where `sample` looks for the last layer's output

    def sample(self, runner, inp) -> torch.Tensor:
        n = inp.num_seqs
        # the last push must have landed from every rank before plain kernels read `gathered`
        # (the bases were advanced by the forward: the last push is at base + 0)
        ew.wait_flags(self.flag_ptr(self.rank, FLAG_AG), self.tp, 0, runner.status,
                      base_ptr=self.epochs.data_ptr() + 4)
        torch.index_select(self.gathered, 0, inp.sample_rows[:n], out=runner.last_rows[:n])
        gemm.linear(runner.last_rows[:n], runner.w.lm_head, acc=runner.logits_acc[:n], status=runner.status)
        if inp.truncation is not None:
            # top-k / top-p: the threshold needs whole rows (gathered here, for the requests that ask
            # for it only); every rank then masks its own shard, and sampling goes on as below
            from daser_b200.engine.sampling import apply_truncation

            local = runner.logits_acc[:n]
            parts = torch.empty(self.tp, n, local.shape[1], dtype=local.dtype, device=self.device)
            dist.all_gather_into_tensor(parts, local.contiguous(), group=self.group)
            whole = parts.permute(1, 0, 2).reshape(n, -1)
            apply_truncation(local, inp.sampling[0], *inp.truncation, whole_rows=whole)
        # (with a temperature the values are Gumbel-perturbed: their maximum over the ranks' shards
        # is the sample, the noise being a function of the seed and the global vocabulary index)
        ew.argmax(runner.logits_acc[:n], runner.best_val[:n], runner.best_idx[:n],
                  index_offset=self.rank * runner.w.vocab_local, zero_after=True, sampling=inp.sampling)
        # one kernel: candidates to every rank by peer stores, arrival counters, bounded wait, pick
        if n > self.cand_cap:
            raise ValueError(f"{n} sequences in one step exceed the sampling table ({self.cand_cap})")
        ew.tp_pick_token(runner.best_val, runner.best_idx, n, self.rank, self.tp, self.cand_cap, self.ptrs["cand"],
                         [self.flag_ptr(r, FLAG_CAND) for r in range(self.tp)], self.epoch_cand, runner.status,
                         runner.best_idx)
        return runner.best_idx[:n]

    def prepare_save_staging(self, geo) -> None:
        """Allocate the symmetric buffer chunks are assembled in (a collective: every rank calls it
        at the same point; engines do so once at start-up)."""
        if self.save_staging is None:
            self.staging_slots = 256
            self.save_staging = self.alloc("save_staging", (self.staging_slots * geo.slot_size,), torch.uint8)

    # -- save: every rank pushes its heads into the owning rank's staging ------------------------------
    def save_step(self, engine, meta) -> None:
        """Store the step's chunks: each chunk is assembled in the staging buffer of the rank that owns
        it (every rank's save kernel compresses its own head slice and writes it there over NVLink),
        and that rank writes the file, fills its tiers and commits."""
        geo = engine.geo
        specs = list(meta.reqs_to_store)
        if not specs:
            return
        self.prepare_save_staging(geo)
        while specs:
            batch, used = [], 0
            while specs and used + len(specs[0].block_ids) <= self.staging_slots:
                s = specs.pop(0)
                batch.append((s, used, engine.owner_of(s.chunk_key)))
                used += len(s.block_ids)
            if not batch:
                raise ValueError("chunk larger than the save staging buffer")
            ptrs, blocks = [], []
            for s, first, owner in batch:
                base = self.ptrs["save_staging"][owner]
                for i, b in enumerate(s.block_ids):
                    ptrs.append(base + (first + i) * geo.slot_size)
                    blocks.append(b)
            engine.kv_backend.save_ptrs(ptrs, blocks)
            torch.cuda.synchronize()
            engine.kv_backend.check_status()
            self.barrier()  # every rank's head slice is in the owner's staging
            wk = engine.worker
            for s, first, owner in batch:
                if owner != self.rank:
                    continue
                n = len(s.block_ids)
                view = self.save_staging[first * geo.slot_size : (first + n) * geo.slot_size]
                wk.transfer.write(view, s.file_offset, n * geo.slot_size)
                for tier in (engine.hbm, engine.host):
                    if tier is not None:
                        tier.admit(s.chunk_key, self.save_staging, first * geo.slot_size, n * geo.slot_size)
                        tier.end_step()
                extra = {"first_block": s.first_block_digest} if s.first_block_digest else {}
                wk._ipc.commit_chunk(s.chunk_key, **extra)
            torch.cuda.synchronize()
            self.barrier()  # staging may be overwritten again; every commit is visible
