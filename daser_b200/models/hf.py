"""Hugging Face checkpoints <-> this package's weight layout (Llama-3 and Qwen3 families).

The reference never touches weights (the remote vLLM loads them); an engine of its own has to.
A checkpoint directory holds ``config.json`` and ``*.safetensors`` shards with the usual names
(``model.layers.N.self_attn.q_proj.weight`` ...).  Here:

* :func:`config_from_hf` reads the architecture into a :class:`LlamaConfig`;
* :func:`weights_from_state_dict` fuses q/k/v and gate/up the way the kernels want them and
  takes a tensor-parallel rank's shard (whole KV heads per rank, the vocabulary split for the
  output projection), from any mapping ``name -> tensor``;
* :func:`load_checkpoint` does the same from a directory, opening the shards lazily so that a rank
  only reads the rows it keeps;
* :func:`state_dict_of` is the inverse for single-rank weights (export, and the round-trip test).

The numerical contract is checked against ``transformers``' own ``LlamaForCausalLM`` and
``Qwen3ForCausalLM`` on small random models (``tests/test_hf_checkpoints.py``): same weights, same
token ids, same logits from ``models/llama.py::reference_forward``.
"""

from __future__ import annotations

import json
import os
from typing import Any, Callable, Mapping, Optional

import torch

from daser_b200.models.llama import LayerWeights, LlamaConfig, LlamaWeights


def config_from_hf(hf: Mapping[str, Any] | Any, name: Optional[str] = None, block_tokens: int = 16) -> LlamaConfig:
    """``hf``: a ``transformers`` config object or the dict of a ``config.json``."""
    get: Callable[[str, Any], Any] = (lambda k, d=None: hf.get(k, d)) if isinstance(hf, Mapping) else (
        lambda k, d=None: getattr(hf, k, d))
    model_type = get("model_type", "llama")
    if model_type not in ("llama", "qwen3"):
        raise ValueError(f"unsupported model_type {model_type!r} (llama and qwen3 are)")
    if get("attention_bias", False) or get("mlp_bias", False):
        raise ValueError("projection biases are not supported")
    heads = int(get("num_attention_heads"))
    hidden = int(get("hidden_size"))
    head_dim = int(get("head_dim", None) or hidden // heads)
    scaling: tuple = ()
    rope = get("rope_scaling", None) or get("rope_parameters", None)
    theta = float(get("rope_theta", None) or (rope or {}).get("rope_theta", 10000.0))
    if rope:
        kind = rope.get("rope_type", rope.get("type", "default"))
        if kind == "llama3":
            scaling = tuple((k, float(rope[k]) if k != "original_max_position_embeddings" else int(rope[k]))
                            for k in ("factor", "low_freq_factor", "high_freq_factor",
                                      "original_max_position_embeddings"))
        elif kind not in ("default", None):
            raise ValueError(f"unsupported rope scaling {kind!r}")
    return LlamaConfig(
        name=name or str(get("_name_or_path", "") or model_type), vocab_size=int(get("vocab_size")), hidden=hidden,
        num_layers=int(get("num_hidden_layers")), num_heads=heads,
        num_kv_heads=int(get("num_key_value_heads", None) or heads), head_dim=head_dim,
        intermediate=int(get("intermediate_size")), rope_theta=theta, rope_scaling=scaling,
        rms_eps=float(get("rms_norm_eps", 1e-5)), block_tokens=block_tokens,
        max_position=int(get("max_position_embeddings", 8192)), qk_norm=model_type == "qwen3",
    )


def _rows(get: Callable[[str, Optional[slice]], torch.Tensor], name: str, lo: int, hi: int) -> torch.Tensor:
    return get(name, slice(lo, hi))


def weights_from_state_dict(cfg: LlamaConfig, tensors: Mapping[str, torch.Tensor] | Callable, tp: int = 1, rank: int = 0,
                            dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu") -> LlamaWeights:
    """``tensors``: a mapping, or ``get(name, row_slice_or_None) -> tensor`` (lazy readers)."""
    if cfg.num_heads % tp or cfg.num_kv_heads % tp or cfg.intermediate % tp or cfg.vocab_size % tp:
        raise ValueError("heads, kv heads, intermediate size and vocabulary must divide by tp")
    if callable(tensors):
        get = tensors
        has = lambda n: True  # noqa: E731  (a lazy reader raises for a missing name)
        try:
            get("lm_head.weight", slice(0, 1))
            tied = False
        except KeyError:
            tied = True
    else:
        sd = tensors
        get = lambda n, s=None: sd[n] if s is None else sd[n][s]  # noqa: E731
        tied = "lm_head.weight" not in sd
        has = lambda n: n in sd  # noqa: E731

    def put(t: torch.Tensor) -> torch.Tensor:
        return t.to(device=device, dtype=dtype).contiguous()

    D = cfg.head_dim
    hq, hkv, inter = cfg.num_heads // tp, cfg.num_kv_heads // tp, cfg.intermediate // tp
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        q = _rows(get, p + "self_attn.q_proj.weight", rank * hq * D, (rank + 1) * hq * D)
        k = _rows(get, p + "self_attn.k_proj.weight", rank * hkv * D, (rank + 1) * hkv * D)
        v = _rows(get, p + "self_attn.v_proj.weight", rank * hkv * D, (rank + 1) * hkv * D)
        gate = _rows(get, p + "mlp.gate_proj.weight", rank * inter, (rank + 1) * inter)
        up = _rows(get, p + "mlp.up_proj.weight", rank * inter, (rank + 1) * inter)
        wo = get(p + "self_attn.o_proj.weight", None)[:, rank * hq * D : (rank + 1) * hq * D]
        down = get(p + "mlp.down_proj.weight", None)[:, rank * inter : (rank + 1) * inter]
        layers.append(LayerWeights(
            input_norm=put(get(p + "input_layernorm.weight", None)),
            wqkv=put(torch.cat([q, k, v])), wo=put(wo),
            post_norm=put(get(p + "post_attention_layernorm.weight", None)),
            w_gate_up=put(torch.cat([gate, up])), w_down=put(down),
            q_norm=put(get(p + "self_attn.q_norm.weight", None)) if cfg.qk_norm else None,
            k_norm=put(get(p + "self_attn.k_norm.weight", None)) if cfg.qk_norm else None,
        ))
    v_loc = cfg.vocab_size // tp
    head_name = "model.embed_tokens.weight" if tied else "lm_head.weight"
    assert has(head_name)
    return LlamaWeights(cfg, tp, rank, put(get("model.embed_tokens.weight", None)), layers,
                        put(get("model.norm.weight", None)),
                        put(_rows(get, head_name, rank * v_loc, (rank + 1) * v_loc)), meta={"tied_head": tied})


def state_dict_of(w: LlamaWeights) -> dict[str, torch.Tensor]:
    """Single-rank weights under the checkpoint's names (gate/up rows in the plain order)."""
    if w.tp != 1:
        raise ValueError("export needs unsharded weights")
    cfg, D = w.cfg, w.cfg.head_dim
    q_end, k_end = cfg.num_heads * D, (cfg.num_heads + cfg.num_kv_heads) * D
    out = {"model.embed_tokens.weight": w.embed, "model.norm.weight": w.final_norm, "lm_head.weight": w.lm_head}
    for i, lw in enumerate(w.layers):
        p = f"model.layers.{i}."
        gu = w.gate_up_plain(lw)
        out.update({
            p + "input_layernorm.weight": lw.input_norm, p + "post_attention_layernorm.weight": lw.post_norm,
            p + "self_attn.q_proj.weight": lw.wqkv[:q_end], p + "self_attn.k_proj.weight": lw.wqkv[q_end:k_end],
            p + "self_attn.v_proj.weight": lw.wqkv[k_end:], p + "self_attn.o_proj.weight": lw.wo,
            p + "mlp.gate_proj.weight": gu[: cfg.intermediate], p + "mlp.up_proj.weight": gu[cfg.intermediate :],
            p + "mlp.down_proj.weight": lw.w_down,
        })
        if cfg.qk_norm:
            out[p + "self_attn.q_norm.weight"] = lw.q_norm
            out[p + "self_attn.k_norm.weight"] = lw.k_norm
    return out


def load_checkpoint(path: str, tp: int = 1, rank: int = 0, dtype: torch.dtype = torch.bfloat16,
                    device: str | torch.device = "cpu", block_tokens: int = 16) -> LlamaWeights:
    """A checkpoint directory (``config.json`` + ``*.safetensors``, sharded or not) -> this rank's weights."""
    from safetensors import safe_open

    with open(os.path.join(path, "config.json")) as f:
        cfg = config_from_hf(json.load(f), name=os.path.basename(os.path.normpath(path)), block_tokens=block_tokens)
    index_file = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index_file):
        with open(index_file) as f:
            where = dict(json.load(f)["weight_map"])
    else:
        where = {}
        for fname in sorted(os.listdir(path)):
            if fname.endswith(".safetensors"):
                with safe_open(os.path.join(path, fname), framework="pt") as sf:
                    where.update({k: fname for k in sf.keys()})
    handles: dict[str, Any] = {}

    def get(name: str, rows: Optional[slice]) -> torch.Tensor:
        if name not in where:
            raise KeyError(name)
        fname = where[name]
        if fname not in handles:
            handles[fname] = safe_open(os.path.join(path, fname), framework="pt").__enter__()
        sl = handles[fname].get_slice(name)
        return sl[:] if rows is None else sl[rows.start : rows.stop]

    try:
        return weights_from_state_dict(cfg, get, tp=tp, rank=rank, dtype=dtype, device=device)
    finally:
        for handle in handles.values():  # the shards were opened lazily and stayed open for the slices
            try:
                handle.__exit__(None, None, None)
            except Exception:
                pass
