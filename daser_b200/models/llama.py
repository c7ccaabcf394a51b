"""Llama-family decoder: configuration, (sharded) weights and a plain-PyTorch forward.

The reference has no model code; its engine is stock vLLM
(``vllm/model_executor/models/llama.py``).  This module defines the architecture once:

* :class:`LlamaConfig` with presets for the toy decoder of the CPU plumbing check,
  Llama-3-8B and Llama-3-70B;
* :class:`LlamaWeights` — random-init weights, already laid out per tensor-parallel rank
  (QKV and gate/up column-sharded by heads / intermediate size, O and down row-sharded);
* :func:`reference_forward` — an fp32 PyTorch forward over a paged KV pool.  It is the
  CPU engine for the plumbing check and the numerical oracle for the CUDA engine
  (:mod:`daser_b200.engine.runner`), which runs the same graph with the hand-written kernels.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from daser_b200.kv import codec
from daser_b200.position.rope_reencoder import inv_freq_table


@dataclass(frozen=True)
class LlamaConfig:
    name: str = "toy"
    vocab_size: int = 32000
    hidden: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate: int = 512
    rope_theta: float = 10000.0
    rope_scaling: tuple = ()  # items of the scaling dict; empty = plain RoPE
    rms_eps: float = 1e-5
    block_tokens: int = 16
    max_position: int = 8192
    # Qwen3 family: RMSNorm over head_dim on every query and key head (one weight vector each per
    # layer, shared by the heads) between the QKV projection and RoPE
    qk_norm: bool = False

    def scaling_dict(self) -> dict[str, Any]:
        return dict(self.rope_scaling)

    def inv_freq(self) -> list[float]:
        return inv_freq_table(self.head_dim, self.rope_theta, self.scaling_dict())

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def param_count(self) -> int:
        per_layer = (
            (self.q_size + 2 * self.kv_size) * self.hidden
            + self.hidden * self.q_size
            + 3 * self.intermediate * self.hidden
            + 2 * self.hidden
        )
        return self.num_layers * per_layer + 2 * self.vocab_size * self.hidden + self.hidden


_LLAMA3_SCALING = (
    ("factor", 8.0),
    ("low_freq_factor", 1.0),
    ("high_freq_factor", 4.0),
    ("original_max_position_embeddings", 8192),
)

PRESETS = {
    # the CPU plumbing check: 2 layers, 4 heads / 2 KV heads, head_dim 64, hidden 256, theta 1e4
    "toy": LlamaConfig(),
    "llama3-8b": LlamaConfig("llama3-8b", 128256, 4096, 32, 32, 8, 128, 14336, 500000.0, _LLAMA3_SCALING,
                             1e-5, 16, 131072),
    "llama3-70b": LlamaConfig("llama3-70b", 128256, 8192, 80, 64, 8, 128, 28672, 500000.0, _LLAMA3_SCALING,
                              1e-5, 16, 131072),
    # small GPU test model with the 70B head geometry
    "tiny-gqa": LlamaConfig("tiny-gqa", 1024, 512, 2, 8, 2, 128, 1024, 500000.0, (), 1e-5, 16, 8192),
    # the same with 8 KV heads, so that it shards 8 ways (2 query heads + 1 KV head per rank)
    "tiny-8kv": LlamaConfig("tiny-8kv", 1024, 1024, 2, 16, 8, 128, 2048, 500000.0, (), 1e-5, 16, 8192),
    # the model of the reference's own end-to-end runs (tests/integration/conftest.py:30 there:
    # 36 layers x 8 KV heads x 128 x 16 tokens x bf16 x 2 = 2 359 296 bytes per slot)
    "qwen3-8b": LlamaConfig("qwen3-8b", 151936, 4096, 36, 32, 8, 128, 12288, 1000000.0, (), 1e-6, 16, 40960, True),
    "toy-qk": LlamaConfig("toy-qk", 32000, 256, 2, 4, 2, 64, 512, 10000.0, (), 1e-6, 16, 8192, True),
    "tiny-gqa-qk": LlamaConfig("tiny-gqa-qk", 1024, 512, 2, 8, 2, 128, 1024, 1000000.0, (), 1e-6, 16, 8192, True),
}


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    wqkv: torch.Tensor  # [(Hq + 2 Hkv) / tp * D, hidden]
    wo: torch.Tensor  # [hidden, Hq / tp * D]
    post_norm: torch.Tensor
    w_gate_up: torch.Tensor  # [2 * I / tp, hidden]: gate rows then up rows
    w_down: torch.Tensor  # [hidden, I / tp]
    q_norm: Optional[torch.Tensor] = None  # [head_dim], models with qk_norm only (replicated)
    k_norm: Optional[torch.Tensor] = None


@dataclass
class LlamaWeights:
    cfg: LlamaConfig
    tp: int
    rank: int
    embed: torch.Tensor  # [vocab, hidden] (replicated)
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor  # [vocab / tp, hidden]
    meta: dict = field(default_factory=dict)
    # 0: w_gate_up rows are [gate | up].  b > 0: blocks of b gate rows followed by the matching up
    # rows (the order in which a GEMM tile holds both halves, so SwiGLU can be its epilogue).
    gate_up_block: int = 0

    def interleave_gate_up_(self, block: int = 64) -> "LlamaWeights":
        """Reorder every layer's gate/up rows in place (one layer-sized temporary at a time)."""
        if self.gate_up_block == block:
            return self
        if self.gate_up_block != 0 or self.inter_local % block:
            raise ValueError("gate/up rows cannot be interleaved in blocks of %d" % block)
        for lw in self.layers:
            if lw.w_gate_up is None:  # a layer another pipeline stage runs
                continue
            two_i, hidden = lw.w_gate_up.shape
            src = lw.w_gate_up.view(2, two_i // 2 // block, block, hidden).transpose(0, 1)
            lw.w_gate_up.copy_(src.reshape(two_i, hidden).clone())
        self.gate_up_block = block
        return self

    def gate_up_plain(self, lw: "LayerWeights") -> torch.Tensor:
        """``lw.w_gate_up`` as [gate | up] whatever the stored order (oracles; copies when interleaved)."""
        b = self.gate_up_block
        if b == 0:
            return lw.w_gate_up
        two_i, hidden = lw.w_gate_up.shape
        return lw.w_gate_up.view(two_i // 2 // b, 2, b, hidden).transpose(0, 1).reshape(two_i, hidden)

    @property
    def heads_local(self) -> int:
        return self.cfg.num_heads // self.tp

    @property
    def kv_heads_local(self) -> int:
        return max(1, self.cfg.num_kv_heads // self.tp)

    @property
    def inter_local(self) -> int:
        return self.cfg.intermediate // self.tp

    @property
    def vocab_local(self) -> int:
        return self.cfg.vocab_size // self.tp

    @classmethod
    def random(cls, cfg: LlamaConfig, device: str | torch.device = "cpu", dtype: torch.dtype = torch.float32,
               tp: int = 1, rank: int = 0, seed: int = 0, std: float = 0.02,
               layers: Optional[range] = None) -> "LlamaWeights":
        """Random-init weights for ``rank`` of ``tp``.

        ``layers`` keeps only that range of layers (a pipeline stage): the others get their norm
        weights and no matrices, and every tensor that IS generated equals the one the full model
        would hold (seeds are per tensor).

        Tensors are filled in place on ``device`` (no full-size temporaries), so the 70B
        model initialises inside one 180 GB GPU.  Every rank seeds per tensor from
        ``(seed, tensor index)`` and generates only its own shard.
        """
        if cfg.num_heads % tp or cfg.intermediate % tp or cfg.vocab_size % tp:
            raise ValueError("heads, intermediate size and vocabulary must divide by tp")
        if cfg.num_kv_heads % tp and tp % cfg.num_kv_heads:
            raise ValueError("kv heads and tp must divide one another")
        gen = torch.Generator(device=device)
        counter = [0]

        def mat(rows: int, cols: int, shard: bool = True) -> torch.Tensor:
            counter[0] += 1
            gen.manual_seed(seed * 1_000_003 + counter[0] * 97 + (rank if shard else 0))
            t = torch.empty((rows, cols), dtype=dtype, device=device)
            t.normal_(0.0, std, generator=gen)
            return t

        def ones(n: int) -> torch.Tensor:
            return torch.ones(n, dtype=dtype, device=device)

        D = cfg.head_dim
        hq, hkv = cfg.num_heads // tp, max(1, cfg.num_kv_heads // tp)
        inter = cfg.intermediate // tp
        embed = mat(cfg.vocab_size, cfg.hidden, shard=False)

        def head_norm() -> torch.Tensor:  # near one, not one: a misapplied weight must show in tests
            counter[0] += 1
            gen.manual_seed(seed * 1_000_003 + counter[0] * 97)
            t = torch.empty(D, dtype=dtype, device=device)
            t.normal_(1.0, 0.1, generator=gen)
            return t

        keep = layers
        layers = []
        for li in range(cfg.num_layers):
            if keep is not None and li not in keep:
                counter[0] += 4 + (2 if cfg.qk_norm else 0)  # the tensors this layer would have drawn
                layers.append(LayerWeights(ones(cfg.hidden), None, None, ones(cfg.hidden), None, None))
                continue
            layers.append(
                LayerWeights(
                    input_norm=ones(cfg.hidden),
                    wqkv=mat((hq + 2 * hkv) * D, cfg.hidden),
                    wo=mat(cfg.hidden, hq * D),
                    post_norm=ones(cfg.hidden),
                    w_gate_up=mat(2 * inter, cfg.hidden),
                    w_down=mat(cfg.hidden, inter),
                    q_norm=head_norm() if cfg.qk_norm else None,
                    k_norm=head_norm() if cfg.qk_norm else None,
                )
            )
        return cls(cfg, tp, rank, embed, layers, ones(cfg.hidden), mat(cfg.vocab_size // tp, cfg.hidden))


def shard_weights(full: LlamaWeights, tp: int, rank: int) -> LlamaWeights:
    """Rank ``rank``'s shard of single-rank weights (tests compare TP against TP=1 this way)."""
    cfg = full.cfg
    assert full.tp == 1 and cfg.num_kv_heads % tp == 0
    assert full.gate_up_block == 0, "shard the plain layout, then interleave the shard"
    D = cfg.head_dim
    hq, hkv, inter = cfg.num_heads // tp, cfg.num_kv_heads // tp, cfg.intermediate // tp
    q_end, k_end = cfg.num_heads * D, (cfg.num_heads + cfg.num_kv_heads) * D
    layers = []
    for lw in full.layers:
        q = lw.wqkv[rank * hq * D : (rank + 1) * hq * D]
        k = lw.wqkv[q_end + rank * hkv * D : q_end + (rank + 1) * hkv * D]
        v = lw.wqkv[k_end + rank * hkv * D : k_end + (rank + 1) * hkv * D]
        gate = lw.w_gate_up[rank * inter : (rank + 1) * inter]
        up = lw.w_gate_up[cfg.intermediate + rank * inter : cfg.intermediate + (rank + 1) * inter]
        layers.append(
            LayerWeights(
                input_norm=lw.input_norm,
                wqkv=torch.cat([q, k, v]).contiguous(),
                wo=lw.wo[:, rank * hq * D : (rank + 1) * hq * D].contiguous(),
                post_norm=lw.post_norm,
                w_gate_up=torch.cat([gate, up]).contiguous(),
                w_down=lw.w_down[:, rank * inter : (rank + 1) * inter].contiguous(),
                q_norm=lw.q_norm, k_norm=lw.k_norm,
            )
        )
    v_loc = cfg.vocab_size // tp
    return LlamaWeights(cfg, tp, rank, full.embed, layers, full.final_norm,
                        full.lm_head[rank * v_loc : (rank + 1) * v_loc].contiguous())


class TorchPagedKV:
    """Head-major paged pool ``[L, N, 2, H, B, D]`` in a torch dtype (the CPU engine's pool)."""

    def __init__(self, cfg: LlamaConfig, num_blocks: int, dtype: torch.dtype = torch.float32,
                 device: str | torch.device = "cpu", kv_heads: Optional[int] = None,
                 num_layers: Optional[int] = None) -> None:
        self.cfg = cfg
        self.num_blocks = num_blocks
        self.kv_heads = kv_heads or cfg.num_kv_heads
        # num_layers: a pipeline stage keeps only its own layers' KV
        self.data = torch.zeros(
            num_layers or cfg.num_layers, num_blocks, 2, self.kv_heads, cfg.block_tokens, cfg.head_dim, dtype=dtype, device=device
        )

    def write(self, layer: int, block_ids: torch.Tensor, offsets: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """``k, v``: ``[T, H, D]`` go to ``(block_ids[t], offsets[t])``."""
        self.data[layer, block_ids, 0, :, offsets] = k.to(self.data.dtype)
        self.data[layer, block_ids, 1, :, offsets] = v.to(self.data.dtype)

    def gather(self, layer: int, block_table: torch.Tensor, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        """K and V ``[length, H, D]`` of a sequence whose blocks are ``block_table``."""
        blk = self.data[layer, block_table]  # [nb, 2, H, B, D]
        kv = blk.permute(1, 0, 3, 2, 4).reshape(2, -1, self.kv_heads, self.cfg.head_dim)
        return kv[0, :length], kv[1, :length]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


@torch.no_grad()
def reference_forward(
    weights: LlamaWeights,
    tokens: torch.Tensor,
    positions: torch.Tensor,
    pool: TorchPagedKV,
    block_table: torch.Tensor,
    context_len: int,
    return_logits: bool = True,
    layers: Optional[range] = None,
    hidden_in: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Run ``tokens`` (at ``positions``) of ONE sequence through the model.

    ``layers`` restricts the pass to a contiguous range of decoder layers (a pipeline stage):
    a range that does not start at 0 takes its input from ``hidden_in`` instead of the
    embedding, a range that does not end at the last layer returns the residual stream
    ``[T, hidden]`` (fp32) without the final norm, and ``pool`` then holds only the stage's own
    layers (layer ``i`` of the model is pool layer ``i - layers.start``).

    The sequence already has ``context_len`` tokens cached in ``pool`` (written earlier or
    restored by the connector); the new tokens occupy cache slots ``context_len ..``.
    K/V of the new tokens are written to the pool, attention is causal over cache + new
    tokens.  Returns logits ``[T, vocab]`` (or the final hidden states).  Single rank only
    (``weights.tp == 1``): this is the oracle, not the parallel engine.
    """
    cfg = weights.cfg
    assert weights.tp == 1
    T = tokens.numel()
    D, Hq, Hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    dev = weights.embed.device
    cos, sin = codec.rope_cos_sin(positions.cpu(), cfg.inv_freq())
    cos, sin = cos.to(dev), sin.to(dev)
    slots = torch.arange(context_len, context_len + T, device=dev)
    blk = block_table.to(dev)[slots // cfg.block_tokens]
    off = slots % cfg.block_tokens
    total = context_len + T
    stage = layers if layers is not None else range(len(weights.layers))
    if stage.start == 0:
        h = weights.embed[tokens.to(dev).long()].float()
    else:
        assert hidden_in is not None and hidden_in.shape == (T, cfg.hidden)
        h = hidden_in.to(dev).float()
    for li, lw in ((i - stage.start, weights.layers[i]) for i in stage):
        x = rms_norm(h, lw.input_norm, cfg.rms_eps)
        qkv = x @ lw.wqkv.float().t()
        q = qkv[:, : Hq * D].reshape(T, Hq, D)
        k = qkv[:, Hq * D : (Hq + Hkv) * D].reshape(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D :].reshape(T, Hkv, D)
        if cfg.qk_norm:
            q = rms_norm(q, lw.q_norm, cfg.rms_eps)
            k = rms_norm(k, lw.k_norm, cfg.rms_eps)
        q = codec.rope_rotate(q, cos, sin)
        k = codec.rope_rotate(k, cos, sin)
        pool.write(li, blk, off, k, v)
        k_all, v_all = pool.gather(li, block_table.to(dev), total)
        k_all = k_all.float().repeat_interleave(Hq // Hkv, dim=1)
        v_all = v_all.float().repeat_interleave(Hq // Hkv, dim=1)
        scores = torch.einsum("thd,shd->hts", q, k_all) / (D**0.5)
        key_pos = torch.arange(total, device=dev)
        mask = key_pos[None, :] > (context_len + torch.arange(T, device=dev))[:, None]
        scores = scores.masked_fill(mask[None], float("-inf"))
        attn = torch.einsum("hts,shd->thd", scores.softmax(-1), v_all).reshape(T, Hq * D)
        h = h + attn @ lw.wo.float().t()
        x = rms_norm(h, lw.post_norm, cfg.rms_eps)
        gu = x @ weights.gate_up_plain(lw).float().t()
        inter = gu.shape[1] // 2
        h = h + (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]) @ lw.w_down.float().t()
    if stage.stop != len(weights.layers):
        return h
    h = rms_norm(h, weights.final_norm, cfg.rms_eps)
    if not return_logits:
        return h
    return h @ weights.lm_head.float().t()
