"""CUDA runner and GPU RAG engine against the fp32 PyTorch reference model."""

import random

import pytest
import torch

from conftest import LiveControlPlane
from daser_b200.models.llama import PRESETS, LlamaWeights, TorchPagedKV, reference_forward

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("interleave", [False, True])
def test_runner_matches_reference_forward(interleave):
    from daser_b200.engine.runner import GpuModelRunner, make_step_inputs

    cfg = PRESETS["tiny-gqa"]
    w = LlamaWeights.random(cfg, "cuda", torch.bfloat16, seed=3, std=0.05)
    if interleave:
        w.interleave_gate_up_()  # the row order the engine uses (SwiGLU as the GEMM epilogue)
    runner = GpuModelRunner(cfg, w, num_blocks=64, max_tokens=64)
    rng = random.Random(0)
    tokens = [rng.randrange(cfg.vocab_size) for _ in range(40)]
    table = [5, 9, 2, 30]
    inp = make_step_inputs([{"tokens": tokens[:33], "start_pos": 0, "block_table": table}], 16, "cuda")
    runner.forward(inp)
    inp2 = make_step_inputs([{"tokens": tokens[33:], "start_pos": 33, "block_table": table}], 16, "cuda")
    logits = runner.logits(inp2)
    runner.check_status()
    # reference: same weights in fp32 on the CPU, bf16 pool emulated in fp32
    wf = LlamaWeights(cfg, 1, 0, w.embed.float().cpu(),
                      [type(l)(*(t.float().cpu() for t in (l.input_norm, l.wqkv, l.wo, l.post_norm, l.w_gate_up, l.w_down)))
                       for l in w.layers], w.final_norm.float().cpu(), w.lm_head.float().cpu(),
                      gate_up_block=w.gate_up_block)
    pool = TorchPagedKV(cfg, 64)
    reference_forward(wf, torch.tensor(tokens[:33]), torch.arange(33), pool, torch.tensor(table), 0, return_logits=False)
    ref = reference_forward(wf, torch.tensor(tokens[33:]), torch.arange(33, 40), pool, torch.tensor(table), 33)
    got = logits.float().cpu()[0]
    want = ref[-1]
    # bf16 activations + fp8 KV against fp32: compare direction and top token
    cos = torch.nn.functional.cosine_similarity(got, want, dim=0).item()
    assert cos > 0.98, cos
    assert (got - want).abs().max().item() < 0.15 * want.abs().max().item() + 0.05


def test_gpu_rag_engine_restored_equals_recomputed(tmp_path):
    from daser_b200.engine.rag_gpu import GpuRagEngine
    from daser_b200.kv import codec

    cfg = PRESETS["tiny-gqa"]
    lp = LiveControlPlane(tmp_path, total_slots=256,
                          slot_size=cfg.num_layers * 2 * 16 * cfg.num_kv_heads * cfg.head_dim * 5 // 4).start()
    eng = GpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=256, max_tokens=128, hbm_slots=64)
    try:
        rng = random.Random(1)
        chunks = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (64, 128, 48)]
        for c in chunks:
            eng.store_chunk(c)
        query = [rng.randrange(cfg.vocab_size) for _ in range(20)]
        # cold: from the store file; warm: from the HBM tier; both must restore all chunks
        for attempt in range(2):
            seen = []
            req = eng.generate([chunks[2], chunks[0], chunks[1]], query, max_new_tokens=4, on_token=seen.append)
            assert req.restored_chunks == 3 and len(req.generated) == 4
            assert seen == [int(t) for t in req.generated]  # reported token by token, as sampled
            assert req.ttft_ms > 0 and req.ttft_device_ms > 0
        # restored + rotated KV equals KV recomputed at the new offset (up to fp8 requantisation)
        from daser_b200.engine.rag_gpu import RagRequest

        r = eng.submit(RagRequest([chunks[2], chunks[0]], query, 2))  # stays running: blocks are kept
        eng._ttft_step(eng.waiting.pop(0))
        off = len(chunks[2])
        blocks_restored = r.block_table[off // 16 : (off + 64) // 16]
        fresh = eng.blocks.alloc(4)
        eng._prefill_tokens(chunks[0], off, [0] * (off // 16) + fresh)  # same positions, fresh blocks
        torch.cuda.synchronize()
        pay, sc = eng.runner.kv_payload.cpu(), eng.runner.kv_scales.cpu()
        got = codec.dequantize_fp8b16(pay[:, blocks_restored], sc[:, blocks_restored])
        want = codec.dequantize_fp8b16(pay[:, fresh], sc[:, fresh])
        # layer 0 keys/values depend only on the token and its position: must agree closely
        err0 = (got[0] - want[0]).abs().max().item() / want[0].abs().max().item()
        assert err0 < 0.15, err0
    finally:
        eng.close()
        lp.stop()


def test_batched_decode_matches_one_at_a_time(tmp_path):
    """Continuous batching: three requests decoded together produce the tokens each produces alone."""
    from daser_b200.engine.rag_gpu import GpuRagEngine, RagRequest

    cfg = PRESETS["tiny-gqa"]
    lp = LiveControlPlane(tmp_path, total_slots=256,
                          slot_size=cfg.num_layers * 2 * 16 * cfg.num_kv_heads * cfg.head_dim * 5 // 4).start()
    eng = GpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=256, max_tokens=128, max_seqs=8,
                       hbm_slots=64, host_slots=64)
    try:
        rng = random.Random(2)
        chunk = [rng.randrange(cfg.vocab_size) for _ in range(64)]
        eng.store_chunk(chunk)
        queries = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (5, 17, 9)]
        alone = [eng.generate([chunk], q, max_new_tokens=6).generated for q in queries]
        reqs = [eng.submit(RagRequest([list(chunk)], list(q), 6)) for q in queries]
        while eng.has_work():
            eng.step()
        assert [r.generated for r in reqs] == alone
        assert all(r.done and r.restored_chunks == 1 for r in reqs)
        assert eng.blocks.num_free == 256  # every block came back
        eng.runner.check_status()
    finally:
        eng.close()
        lp.stop()


def test_engine_loop_on_the_gpu_engine_matches_one_request_at_a_time(tmp_path):
    """The serving loop (one thread steps the engine, callers on other threads share its steps)
    around the CUDA engine: concurrent requests decode as one batch, stream their tokens, and
    produce what each produces alone; an abort frees the request's blocks."""
    from daser_b200.engine.loop import EngineLoop
    from daser_b200.engine.rag_gpu import GpuRagEngine, RagRequest

    cfg = PRESETS["tiny-gqa"]
    lp = LiveControlPlane(tmp_path, total_slots=256,
                          slot_size=cfg.num_layers * 2 * 16 * cfg.num_kv_heads * cfg.head_dim * 5 // 4).start()
    eng = GpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=256, max_tokens=128, max_seqs=8,
                       hbm_slots=64, host_slots=64)
    try:
        rng = random.Random(7)
        chunks = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (32, 64, 48)]
        for c in chunks:
            eng.store_chunk(c)
        reqs = [([chunks[i % 3], chunks[(i + 1) % 3]], [rng.randrange(cfg.vocab_size) for _ in range(5 + i)])
                for i in range(5)]
        want = [eng.generate(c, q, max_new_tokens=6).generated for c, q in reqs]
        free = eng.blocks.num_free
        loop = EngineLoop(eng)
        try:
            streams = [[] for _ in reqs]
            futs = [loop.submit(c, q, 6, on_token=streams[i].append) for i, (c, q) in enumerate(reqs)]
            done = [f.result(120) for f in futs]
        finally:
            loop.close()
        eng.runner.check_status()
        assert [r.generated for r in done] == want
        assert streams == want and all(r.restored_chunks == 2 for r in done)
        assert loop.max_batch > 1 and eng.blocks.num_free == free
        # a temperature changes the draw, reproducibly per seed
        a = eng.generate(*reqs[0], max_new_tokens=6, temperature=0.9, seed=5, top_k=8, top_p=0.95).generated
        b = eng.generate(*reqs[0], max_new_tokens=6, temperature=0.9, seed=5, top_k=8, top_p=0.95).generated
        assert a == b and len(a) == 6
        # abort of a running request returns its blocks
        r = eng.submit(RagRequest(reqs[1][0], reqs[1][1], 50))
        eng.step()
        assert r in eng.running and eng.abort(r.req_id) and r.done and eng.blocks.num_free == free
    finally:
        eng.close()
        lp.stop()


def test_missed_chunks_stored_write_behind_are_restored_by_later_requests(tmp_path):
    """``store_misses`` with write-behind stores: a request's missed chunks and its query go through
    the model as one run, the chunk at offset 0 is stored from the request's blocks with the file
    write in flight when the call returns, and a later request that asks for it finds it (the
    engine completes a pending store of a chunk it is asked for before it plans)."""
    from daser_b200.engine.rag_gpu import GpuRagEngine

    cfg = PRESETS["tiny-gqa"]
    lp = LiveControlPlane(tmp_path, total_slots=256,
                          slot_size=cfg.num_layers * 2 * 16 * cfg.num_kv_heads * cfg.head_dim * 5 // 4).start()
    eng = GpuRagEngine(cfg, lp.socket_path, lp.cfg.store_path, num_blocks=256, max_tokens=128, host_slots=64,
                       write_behind=True)
    try:
        rng = random.Random(4)
        a, b = ([rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (64, 48))
        query = [rng.randrange(cfg.vocab_size) for _ in range(7)]
        cold = eng.generate([a, b], query, max_new_tokens=3, store_misses=True)
        assert cold.restored_chunks == 0
        # a (offset 0) was stored in place and may still be in flight; b was recomputed alone and
        # stored through store_chunk, which returns with the chunk visible
        warm = eng.generate([a, b], query, max_new_tokens=3, store_misses=True)
        assert warm.restored_chunks == 2 and not eng.worker.pending_store_keys()
        assert len(warm.generated) == 3
        other = eng.generate([b, a], query, max_new_tokens=2)
        assert other.restored_chunks == 2
        eng.runner.check_status()
        assert eng.blocks.num_free == 256
    finally:
        eng.close()
        lp.stop()
