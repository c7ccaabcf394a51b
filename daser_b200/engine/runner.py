"""CUDA model runner: the Llama forward on the hand-written sm_100a kernels.

The reference has no engine (stock vLLM's ``GPUModelRunner`` plays this part).  One
:class:`GpuModelRunner` lives in each process (one process per GPU).  It owns

* this rank's weight shards (bf16),
* this rank's slice of the paged KV pool: block-scaled fp8, head-major
  ``[layer, block, k|v, head, token, dim]`` payload plus fp32 scales, which is what the fused
  restore kernel writes into and the attention kernel reads from,
* persistent activation buffers, so a step allocates nothing.

Per layer the step is: tcgen05 GEMM (QKV) -> RoPE + KV write -> fp8 paged attention ->
tcgen05 GEMM (O) -> add + RMSNorm -> tcgen05 GEMM (gate, up) -> SwiGLU -> tcgen05 GEMM (down)
-> add + RMSNorm.  Skinny GEMMs run split-K into fp32 accumulators that the consuming kernel
reads and hands back zeroed.

Tensor parallelism (``tp > 1``) follows the sequence-parallel formulation: activations
between blocks are sharded by rows.  The row-parallel GEMMs (O, down) reduce-scatter in their
epilogue straight into the owning rank's accumulator over NVLink; the add + RMSNorm kernel
waits for the arrivals, normalises its rows and pushes them into every rank's gathered
activation buffer; the following column-parallel GEMM is gated on those pushes.  No NCCL call
is made on that path (:mod:`daser_b200.parallel.tp` holds the symmetric buffers and counters).
"""

from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Any, Optional

import torch

from daser_b200.kv.layout import KVGeometry
from daser_b200.models.llama import LlamaConfig, LlamaWeights
from daser_b200.ops import _lib, attention, elementwise as ew, gemm, kv_ops


@dataclass
class StepInputs:
    """Device tensors describing one engine step (all int32 unless noted)."""

    tokens: torch.Tensor  # [T]
    positions: torch.Tensor  # [T]
    slot_mapping: torch.Tensor  # [T] int64: block * block_tokens + offset
    block_tables: torch.Tensor  # [num_seqs, max_blocks]
    q_start: torch.Tensor  # [num_seqs + 1]
    ctx_lens: torch.Tensor  # [num_seqs]
    sample_rows: torch.Tensor  # [num_seqs] row index of each sequence's last token
    num_tokens: int
    num_seqs: int
    max_q_len: int
    max_ctx: int
    persistent: bool = False  # tensors are the runner's own fixed buffers (graph replay is allowed)
    # (inv_temp float32[num_seqs], seeds int64[num_seqs]) when a sequence of the step samples with a
    # temperature; None = every sequence is greedy
    sampling: Optional[tuple] = None
    # (top_k int64[num_seqs], top_p float32[num_seqs]) when a sampling sequence also truncates
    truncation: Optional[tuple] = None


def split_layers(num_layers: int, parts: int) -> list[tuple[int, int]]:
    """``num_layers`` cut into at most ``parts`` consecutive runs of near-equal length."""
    parts = max(1, min(int(parts), num_layers))
    base, extra = divmod(num_layers, parts)
    out, first = [], 0
    for i in range(parts):
        n = base + (1 if i < extra else 0)
        out.append((first, n))
        first += n
    return out


_BUCKET_ROWS = os.environ.get("DASER_BUCKET_ROWS", "1") != "0"


class GpuModelRunner:
    def __init__(self, cfg: LlamaConfig, weights: LlamaWeights, num_blocks: int, max_tokens: int = 256,
                 max_seqs: int = 64, tp_ctx=None, device: Optional[torch.device] = None,
                 max_blocks: int = 512, use_graphs: bool = True, layer_groups: int = 8,
                 layer_range: Optional[range] = None, pool_layers: Optional[int] = None, pp_link=None) -> None:
        self.cfg = cfg
        self.w = weights
        # pipeline stage: the layers this process runs, its links to the neighbouring stages
        # (``parallel/pp.py::StageLink``) and how many layers its pool and slot images have room for
        self.layers = layer_range if layer_range is not None else range(cfg.num_layers)
        self.pp_link = pp_link
        if pp_link is not None and tp_ctx is not None:
            raise ValueError("a pipeline stage runs on one GPU here (no tensor parallelism inside a stage)")
        self.tp = weights.tp
        self.rank = weights.rank
        self.tp_ctx = tp_ctx
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.num_blocks = num_blocks
        D, B = cfg.head_dim, cfg.block_tokens
        self.hq = weights.heads_local
        self.hkv = weights.kv_heads_local
        dev = self.device

        # ---- paged KV pool (this rank's heads) ----
        n_pool_layers = pool_layers if pool_layers is not None else len(self.layers)
        if n_pool_layers < len(self.layers):
            raise ValueError("the pool has fewer layers than the stage runs")
        shape = (n_pool_layers, num_blocks, 2, self.hkv, B, D)
        if tp_ctx is not None:
            self.kv_payload = tp_ctx.alloc("kv_payload", shape, torch.uint8)
            self.kv_scales = tp_ctx.alloc("kv_scales", shape[:-1] + (D // 16,), torch.float32)
            self.kv_payload.zero_()
            self.kv_scales.fill_(1.0)
        else:
            self.kv_payload = torch.zeros(shape, dtype=torch.uint8, device=dev)
            self.kv_scales = torch.ones(shape[:-1] + (D // 16,), dtype=torch.float32, device=dev)
        self.local_pool = kv_ops.PagedKVPool.from_tensors([self.kv_payload], [self.kv_scales], "LNKHTD")
        # geometry of a stored slot: ALL kv heads, fp8b16
        self.geo = KVGeometry(n_pool_layers, cfg.num_kv_heads, D, B, 2, "fp8b16")
        self.cos_sin = kv_ops.rope_table(min(cfg.max_position, 32768), cfg.inv_freq(), dev)

        # ---- activation buffers ----
        T, H = max_tokens, cfg.hidden
        qkv_n = (self.hq + 2 * self.hkv) * D
        bf, f32 = torch.bfloat16, torch.float32
        self.h = torch.zeros(T, H, dtype=bf, device=dev)  # residual stream
        self.normed = torch.zeros(T, H, dtype=bf, device=dev)
        self.qkv_acc = torch.zeros(T, qkv_n, dtype=f32, device=dev)
        self.qkv_bf = torch.zeros(T, qkv_n, dtype=bf, device=dev)
        self.q_rot = torch.zeros(T, self.hq, D, dtype=bf, device=dev)
        self.attn_out = torch.zeros(T, self.hq * D, dtype=bf, device=dev)
        self.hid_acc = torch.zeros(T, H, dtype=f32, device=dev)
        self.hid_bf = torch.zeros(T, H, dtype=bf, device=dev)
        inter = weights.inter_local
        self.gu_acc = torch.zeros(T, 2 * inter, dtype=f32, device=dev)
        self.gu_bf = torch.zeros(T, 2 * inter, dtype=bf, device=dev)
        self.act = torch.zeros(T, inter, dtype=bf, device=dev)
        self.last_rows = torch.zeros(max_seqs, H, dtype=bf, device=dev)
        self.logits_acc = torch.zeros(max_seqs, weights.vocab_local, dtype=f32, device=dev)
        self.best_val = torch.zeros(max_seqs, dtype=f32, device=dev)
        self.best_idx = torch.zeros(max_seqs, dtype=torch.int32, device=dev)
        self.attn_ws = attention.AttentionWorkspace(dev)
        self.attn_ws.ensure(attention.MAX_ROW_SPLITS, 1, D)  # sized once: captured graphs keep its address
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.tile_counters = torch.zeros(4096, dtype=torch.int32, device=dev)  # split-K "last CTA of a tile" counts
        import os as _os

        # Fused epilogues that finish another operator's work inside the GEMM (RoPE + KV write behind
        # the QKV projection, SwiGLU under split-K).  Both are correct and tested, and both are OFF by
        # default: at serving shapes these GEMMs run split-K, the fused work then falls to the one CTA
        # that completes a tile, and measured on the 70B 64-token step that serial tail costs more
        # than the launch it saves (all-warm TTFT 30.8 ms fused against 30.3 ms with the two kernels).
        self.fuse_qkv_rope = (gemm.can_fuse_qkv_rope(D, cfg.qk_norm) and _os.environ.get("DASER_FUSE_QKV_ROPE", "0") == "1"
                              and -(-max_tokens // 128) * -(-qkv_n // 128) <= self.tile_counters.numel())
        self.fuse_swiglu_split = _os.environ.get("DASER_FUSE_SWIGLU_SPLIT", "0") == "1"
        self.softmax_scale = D**-0.5
        # ---- persistent step inputs (pinned host mirror + device copy) ----
        self.max_blocks = max_blocks
        i32, i64 = torch.int32, torch.int64
        self._in_dev = {
            "tokens": torch.zeros(T, dtype=i32, device=dev), "positions": torch.zeros(T, dtype=i32, device=dev),
            "slot_mapping": torch.zeros(T, dtype=i64, device=dev),
            "block_tables": torch.zeros(max_seqs, max_blocks, dtype=i32, device=dev),
            "q_start": torch.zeros(max_seqs + 1, dtype=i32, device=dev),
            "ctx_lens": torch.zeros(max_seqs, dtype=i32, device=dev),
            "sample_rows": torch.zeros(max_seqs, dtype=i64, device=dev),
        }
        self._in_host = {k: torch.zeros_like(v, device="cpu").pin_memory() for k, v in self._in_dev.items()}
        self._in_event: Optional[torch.cuda.Event] = None
        # ---- CUDA graphs of the forward, one per step shape ----
        self.use_graphs = use_graphs
        self._graphs: dict[tuple, Any] = {}
        self._seen: dict[tuple, int] = {}
        # consecutive runs of layers a step is launched in (see `forward`): [(first layer, count)]
        self.layer_groups = [(self.layers.start + a, n) for a, n in split_layers(len(self.layers), layer_groups)]

    # -- helpers ---------------------------------------------------------------------------------
    def _linear(self, x: torch.Tensor, w: torch.Tensor, acc: torch.Tensor, out_bf: torch.Tensor):
        """``x @ w.T``; returns (tensor, is_fp32_accumulator)."""
        M = x.shape[0]
        bn, ks = gemm.plan_tiles(M, w.shape[0], w.shape[1], allow_split=True)
        if ks > 1:
            gemm.linear(x, w, acc=acc[:M], block_n=bn, k_splits=ks, status=self.status)
            return acc[:M], True
        gemm.linear(x, w, out=out_bf[:M], block_n=bn, k_splits=1, status=self.status)
        return out_bf[:M], False

    def qk_norm(self, lw):
        """The per-head norm of models that have one, as ``ops.elementwise.rope_kv_write`` takes it."""
        if not self.cfg.qk_norm:
            return None
        return (lw.q_norm, lw.k_norm, self.cfg.rms_eps)

    def qkv_rope(self, x: torch.Tensor, lw, inp: "StepInputs", T: int, pool_layer: int, **gate) -> None:
        """QKV projection, RoPE and the KV-cache write: ``self.q_rot[:T]`` holds the rotated queries,
        the step's keys and values are in the paged pool.  One kernel (the GEMM's epilogue does the
        rest) when a 128-column tile is a head and the model has no per-head norm, else GEMM + kernel."""
        D, B = self.cfg.head_dim, self.cfg.block_tokens
        if self.fuse_qkv_rope:
            gemm.linear_qkv_rope(x, lw.wqkv, inp.positions, inp.slot_mapping, self.cos_sin, self.q_rot[:T], self.hq,
                                 self.hkv, B, self.local_pool, pool_layer, 0, self.qkv_acc, self.tile_counters,
                                 status=self.status, **gate)
            return
        bn, ks = gemm.plan_tiles(T, lw.wqkv.shape[0], lw.wqkv.shape[1], allow_split=True)
        if ks > 1:
            gemm.linear(x, lw.wqkv, acc=self.qkv_acc[:T], block_n=bn, k_splits=ks, status=self.status, **gate)
            qkv, f32 = self.qkv_acc[:T], True
        else:
            gemm.linear(x, lw.wqkv, out=self.qkv_bf[:T], block_n=bn, k_splits=1, status=self.status, **gate)
            qkv, f32 = self.qkv_bf[:T], False
        ew.rope_kv_write(qkv, inp.positions, inp.slot_mapping, self.cos_sin, self.q_rot[:T], self.hq, self.hkv, D, B,
                         self.local_pool, pool_layer, 0, zero_after=f32, qk_norm=self.qk_norm(lw))

    def mlp_up(self, x: torch.Tensor, lw, T: int, **gate) -> torch.Tensor:
        """``silu(x Wg^T) * (x Wu^T)`` into ``self.act[:T]``: one GEMM with the activation as its
        epilogue when the weights are interleaved and the shape runs unsplit, else GEMM + kernel."""
        w = self.w
        n2, k = lw.w_gate_up.shape
        if w.gate_up_block == gemm.GATE_UP_BLOCK and gemm.can_fuse_swiglu(T, n2, k, split_ok=self.fuse_swiglu_split):
            _, ks = gemm.plan_tiles(T, n2, k, allow_split=True)
            return gemm.linear_swiglu(x, lw.w_gate_up, self.act[:T], status=self.status, k_splits=ks,
                                      work=self.gu_acc, tile_counters=self.tile_counters, **gate)
        bn, ks = gemm.plan_tiles(T, lw.w_gate_up.shape[0], lw.w_gate_up.shape[1], allow_split=True)
        if ks > 1:
            gemm.linear(x, lw.w_gate_up, acc=self.gu_acc[:T], block_n=bn, k_splits=ks, status=self.status, **gate)
            gu, f32 = self.gu_acc[:T], True
        else:
            gemm.linear(x, lw.w_gate_up, out=self.gu_bf[:T], block_n=bn, k_splits=1, status=self.status, **gate)
            gu, f32 = self.gu_bf[:T], False
        return ew.swiglu(gu, out=self.act[:T], zero_after=f32, block=w.gate_up_block)

    @staticmethod
    def bucket_rows(n: int) -> int:
        """Rows a step of ``n`` tokens is launched with: exact up to 16 (decode batches, prompt
        tails: few shapes, soon all captured), then multiples of 16 up to 128, of 64 up to 512, of
        128 beyond."""
        if n <= 16 or not _BUCKET_ROWS:
            return n
        step = 16 if n <= 128 else 64 if n <= 512 else 128
        return -(-n // step) * step

    # -- step inputs ---------------------------------------------------------------------------------
    def stage_inputs(self, seqs: list[dict]) -> StepInputs:
        """Write one step's inputs into the runner's fixed buffers (pinned host -> device, one
        copy each) and describe them.  ``seqs`` = ``[{tokens, start_pos, block_table}]``."""
        bt = self.cfg.block_tokens
        h = self._in_host
        if self._in_event is not None:
            self._in_event.synchronize()  # the previous step's copies have read the pinned mirror
        t = 0
        h["q_start"][0] = 0
        max_q = max_ctx = 0
        for i, s in enumerate(seqs):
            n, p0, table = len(s["tokens"]), s["start_pos"], s["block_table"]
            if t + n > self.max_tokens or i >= self.max_seqs or len(table) > self.max_blocks:
                raise ValueError("step exceeds the runner's buffers")
            h["tokens"][t : t + n] = torch.as_tensor(s["tokens"], dtype=torch.int32)
            pos = torch.arange(p0, p0 + n, dtype=torch.int64)
            h["positions"][t : t + n] = pos.to(torch.int32)
            tbl = torch.as_tensor(table, dtype=torch.int64)
            h["slot_mapping"][t : t + n] = tbl[pos // bt] * bt + pos % bt
            h["block_tables"][i, : len(table)] = tbl.to(torch.int32)
            t += n
            h["q_start"][i + 1] = t
            h["ctx_lens"][i] = p0 + n
            h["sample_rows"][i] = t - 1
            max_q, max_ctx = max(max_q, n), max(max_ctx, p0 + n)
        ns = len(seqs)
        # Round the step up to a bucket of rows so that steps of nearby sizes share their CUDA graphs
        # (a prompt tail or a missed chunk can have any length; an unseen shape runs eagerly, several
        # hundred launches from the host).  The extra rows belong to no sequence: they write no KV
        # (slot -1), the attention kernels take their row ranges from `q_start`, nothing samples them.
        real = t
        t = min(self.bucket_rows(t), self.max_tokens)
        if t > real:
            h["tokens"][real:t] = 0
            h["positions"][real:t] = 0
            h["slot_mapping"][real:t] = -1
            max_q = min(self.bucket_rows(max_q), t)
        d = self._in_dev
        for name, count in (("tokens", t), ("positions", t), ("slot_mapping", t), ("q_start", ns + 1),
                            ("ctx_lens", ns), ("sample_rows", ns)):
            d[name][:count].copy_(h[name][:count], non_blocking=True)
        d["block_tables"][:ns].copy_(h["block_tables"][:ns], non_blocking=True)
        if self._in_event is None:
            self._in_event = torch.cuda.Event()
        self._in_event.record()
        self.h2d_bytes = t * 16 + ns * (self.max_blocks * 4 + 20) + 4
        sampling = truncation = None
        if any(s.get("temperature", 0.0) > 0.0 for s in seqs):
            # sampling runs outside the captured layer loop, so these need no fixed buffers
            inv = torch.tensor([1.0 / s["temperature"] if s.get("temperature", 0.0) > 0.0 else 0.0 for s in seqs],
                               dtype=torch.float32)
            seeds = torch.tensor([int(s.get("seed", 0)) & 0x7FFFFFFFFFFFFFFF for s in seqs], dtype=torch.int64)
            sampling = (inv.to(self.device), seeds.to(self.device))
            self.h2d_bytes += ns * 12
            if any(s.get("temperature", 0.0) > 0.0 and (s.get("top_k", 0) > 0 or s.get("top_p", 1.0) < 1.0)
                   for s in seqs):
                truncation = (torch.tensor([int(s.get("top_k", 0)) for s in seqs], dtype=torch.int64).to(self.device),
                              torch.tensor([float(s.get("top_p", 1.0)) for s in seqs]).to(self.device))
                self.h2d_bytes += ns * 12
        return StepInputs(d["tokens"][:t], d["positions"][:t], d["slot_mapping"][:t], d["block_tables"][:ns],
                          d["q_start"][: ns + 1], d["ctx_lens"][:ns], d["sample_rows"][:ns], t, ns, max_q, max_ctx,
                          persistent=True, sampling=sampling, truncation=truncation)

    # -- one step -----------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, inp: StepInputs, gate=None) -> torch.Tensor:
        """Run the model on the step's tokens; returns the greedy next token of every sequence
        (int32 ``[num_seqs]``, on the device).

        The layers run in ``self.layer_groups`` consecutive groups.  ``gate(g)``, if given, is
        called on the host right before group ``g`` is launched and queues on the current stream
        whatever that group has to wait for: this is how a chunk restore that is still reading
        layers 10.. from storage lets layers 0..9 start (``GpuRagEngine._ttft_step``).

        Each group of a step shape seen before is replayed from a CUDA graph (captured on the
        second occurrence): a forward is several hundred short kernels and the host would
        otherwise be the bottleneck at small token counts.
        """
        T = inp.num_tokens
        if T > self.max_tokens or inp.num_seqs > self.max_seqs:
            raise ValueError("step exceeds the runner's buffers")
        group = self.hq // self.hkv
        ctx_bucket = max(2048, 1 << (max(inp.max_ctx, 1) - 1).bit_length())  # powers of two: few graph shapes
        nsplit, split_tokens = attention.plan_splits(inp.num_seqs, self.hkv, inp.max_q_len, group, ctx_bucket,
                                                     self.cfg.block_tokens, rows=T * self.hq)
        body = self._body if self.tp == 1 else (lambda *a: self.tp_ctx.forward_body(self, *a))
        shape = (T, inp.num_seqs, inp.max_q_len, nsplit, split_tokens)
        link = self.pp_link
        if link is not None:
            link.drain()  # the previous step's hand-over has left `self.h`
            if not link.first:
                link.recv_prev_into(self.h[:T])  # the residual stream as the previous stage left it
        graphs_ok = self.use_graphs and inp.persistent
        seen = self._seen.get(shape, 0)
        self._seen[shape] = seen + 1
        for g, (l0, count) in enumerate(self.layer_groups):
            if gate is not None:
                gate(g)
            key = shape + (g,)
            if not graphs_ok:
                body(inp, nsplit, split_tokens, l0, l0 + count)
            elif key in self._graphs:
                graph, n_kernels = self._graphs[key]
                graph.replay()
                _lib.launch_count += n_kernels  # kernels of ours that the replay launched
            elif seen == 0 or len(self._graphs) >= 64 * len(self.layer_groups):
                body(inp, nsplit, split_tokens, l0, l0 + count)  # first sight: eager (also loads every kernel)
            else:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                before = _lib.launch_count
                with torch.cuda.graph(graph):
                    body(inp, nsplit, split_tokens, l0, l0 + count)
                self._graphs[key] = (graph, _lib.launch_count - before)
                graph.replay()
        if link is not None and not link.last:
            link.send_next(self.h[:T])  # asynchronous; only the last stage samples
            return None
        if self.tp > 1:
            return self.tp_ctx.sample(self, inp)
        return self.sample(self.normed[:T], inp)

    def _body(self, inp: StepInputs, nsplit: int, split_tokens: int, l0: int = 0, l1: Optional[int] = None) -> None:
        """Layers ``[l0, l1)`` on one GPU (the embedding in front of layer 0, the final norm behind
        the last layer); leaves ``self.normed`` ready for the next group or for sampling."""
        cfg, w = self.cfg, self.w
        l1 = len(w.layers) if l1 is None else l1
        T = inp.num_tokens
        D, B = cfg.head_dim, cfg.block_tokens
        h = self.h[:T]
        normed = self.normed[:T]
        first = self.layers.start
        if l0 == first:
            if first == 0:
                ew.embedding(inp.tokens, w.embed, out=h)
            # (a later pipeline stage finds the residual stream in `h`, received from its predecessor)
            ew.add_rmsnorm(h, w.layers[first].input_norm, out=normed, eps=cfg.rms_eps)
        for li in range(l0, l1):
            lw = w.layers[li]
            pl = li - first  # layer index inside this stage's pool
            self.qkv_rope(normed, lw, inp, T, pl)
            attn = self.attn_out[:T].view(T, self.hq, D)
            attention.paged_attention(self.q_rot[:T], attn, self.local_pool, pl, inp.block_tables, inp.q_start,
                                      inp.ctx_lens, inp.max_q_len, inp.max_ctx, self.hkv, self.softmax_scale,
                                      self.attn_ws, nsplit=nsplit, split_tokens=split_tokens)
            o, f32 = self._linear(self.attn_out[:T], lw.wo, self.hid_acc, self.hid_bf)
            ew.add_rmsnorm(o, lw.post_norm, residual=h, out=normed, eps=cfg.rms_eps, zero_after=f32)
            self.mlp_up(normed, lw, T)
            d, f32 = self._linear(self.act[:T], lw.w_down, self.hid_acc, self.hid_bf)
            next_norm = w.layers[li + 1].input_norm if li + 1 < len(w.layers) else w.final_norm
            ew.add_rmsnorm(d, next_norm, residual=h, out=normed, eps=cfg.rms_eps, zero_after=f32)

    def sample(self, normed: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        n = inp.num_seqs
        torch.index_select(normed, 0, inp.sample_rows[:n], out=self.last_rows[:n])
        gemm.linear(self.last_rows[:n], self.w.lm_head, acc=self.logits_acc[:n], status=self.status)
        if inp.truncation is not None:  # top-k / top-p: a value threshold per row, then sample as usual
            from daser_b200.engine.sampling import apply_truncation

            apply_truncation(self.logits_acc[:n], inp.sampling[0], *inp.truncation)
        ew.argmax(self.logits_acc[:n], self.best_val[:n], self.best_idx[:n],
                  index_offset=self.rank * self.w.vocab_local, zero_after=True, sampling=inp.sampling)
        return self.best_idx[:n]

    def logits(self, inp: StepInputs) -> torch.Tensor:
        """Full forward returning fp32 logits of the sampled rows (tests; single rank)."""
        assert self.tp == 1
        self.forward(inp)  # leaves `normed` of the last layer in place
        n = inp.num_seqs
        gemm.linear(self.last_rows[:n], self.w.lm_head, acc=self.logits_acc[:n], status=self.status)
        out = self.logits_acc[:n].clone()
        self.logits_acc[:n].zero_()
        return out

    def check_status(self) -> None:
        if int(self.status[0].item()) != 0:
            self.status.zero_()
            raise RuntimeError("a GEMM wait ran out (status word set); the step's output is invalid")
        if attention.tc_status() != 0:
            raise RuntimeError("an attention CTA gave up on a bounded wait; the step's output is invalid")


def make_step_inputs(seqs: list[dict], block_tokens: int, device, max_blocks: Optional[int] = None) -> StepInputs:
    """Build :class:`StepInputs` from ``[{tokens, start_pos, block_table}]``.

    ``start_pos`` is the number of tokens already in the sequence's cache.  Host tensors are
    assembled in pinned memory and copied once.
    """
    toks, pos, slots, q_start, ctx, rows = [], [], [], [0], [], []
    for s in seqs:
        n, p0, table = len(s["tokens"]), s["start_pos"], s["block_table"]
        toks.extend(s["tokens"])
        for i in range(n):
            p = p0 + i
            pos.append(p)
            slots.append(table[p // block_tokens] * block_tokens + p % block_tokens)
        q_start.append(q_start[-1] + n)
        ctx.append(p0 + n)
        rows.append(q_start[-1] - 1)
    mb = max_blocks or max(len(s["block_table"]) for s in seqs)
    tables = torch.zeros(len(seqs), mb, dtype=torch.int32)
    for i, s in enumerate(seqs):
        tables[i, : len(s["block_table"])] = torch.tensor(s["block_table"], dtype=torch.int32)

    def dev(x, dt):
        t = torch.tensor(x, dtype=dt).pin_memory()
        return t.to(device, non_blocking=True)

    return StepInputs(
        tokens=dev(toks, torch.int32), positions=dev(pos, torch.int32), slot_mapping=dev(slots, torch.int64),
        block_tables=tables.pin_memory().to(device, non_blocking=True), q_start=dev(q_start, torch.int32),
        ctx_lens=dev(ctx, torch.int32), sample_rows=dev(rows, torch.int64), num_tokens=len(toks),
        num_seqs=len(seqs), max_q_len=max(len(s["tokens"]) for s in seqs), max_ctx=max(ctx),
    )
