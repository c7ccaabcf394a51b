"""Multi-process host logic on CPU ranks (``gloo``): plan broadcast and multi-part commits,
peer-loss detection, a rank that never joins.  Every failure is made on the host."""

import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(scenario: str, world: int, ranks=None, timeout: int = 120):
    port = _free_port()
    procs = []
    for r in (ranks if ranks is not None else range(world)):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_PORT=str(port), MASTER_ADDR="127.0.0.1",
                   PYTHONUNBUFFERED="1")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "gloo_worker.py"), scenario],
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append((p.returncode, out))
    return outs


def test_two_ranks_store_parts_and_restore_their_heads():
    outs = _launch("parts", 2)
    assert all(rc == 0 for rc, _ in outs), "\n".join(o[-2000:] for _, o in outs)
    assert "PARTS_OK" in outs[0][1]


def test_peer_that_leaves_and_peer_that_dies_are_noticed_between_steps():
    outs = _launch("health", 3)
    assert outs[0][0] == 0, outs[0][1][-2000:]
    assert "HEALTH_OK" in outs[0][1]


def test_followers_replay_the_leaders_engine_calls():
    outs = _launch("serve", 3)
    assert all(rc == 0 for rc, _ in outs), "\n".join(o[-2000:] for _, o in outs)
    assert "SERVE_OK" in outs[0][1]


def test_engine_loop_on_the_leader_is_replayed_exactly_by_real_follower_engines():
    outs = _launch("serve_loop", 3, timeout=180)
    assert all(rc == 0 for rc, _ in outs), "\n".join(o[-2000:] for _, o in outs)
    assert "SERVE_LOOP_OK" in outs[0][1]


def test_pipeline_stages_match_a_single_process():
    for world in (2, 3):
        outs = _launch("pipeline", world, timeout=180)
        assert all(rc == 0 for rc, _ in outs), "\n".join(o[-2000:] for _, o in outs)
        assert "PIPELINE_OK" in outs[0][1]


def test_rank_missing_at_rendezvous_fails_within_the_time_limit():
    outs = _launch("late", 2, ranks=[0], timeout=60)
    assert outs[0][0] == 7, outs[0][1][-2000:]
    assert "RENDEZVOUS_FAILED" in outs[0][1]
