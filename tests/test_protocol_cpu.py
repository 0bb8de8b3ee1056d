"""The communication protocol of the sharded step replayed on the host: correctness against a single-process step,
hazard detection when a barrier is removed, bounded waits under injected faults, and the heartbeat watchdog."""
import numpy as np
import pytest

from dice_embeddings_b200.parallel import protocol_sim as ps
from dice_embeddings_b200.parallel.watchdog import DictStore, Heartbeat, RankFailure


def _problem(NE=37, NR=5, D=8, B=12, seed=0):
    rng = np.random.default_rng(seed)
    E, R = rng.normal(size=(NE, D)) * 0.5, rng.normal(size=(NR, D)) * 0.5
    h, r = rng.integers(0, NE, B), rng.integers(0, NR, B)
    labels = (rng.random((B, NE)) < 0.1).astype(np.float64) * 0.9 + 0.005
    return E, R, h, r, labels


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_sharded_protocol_equals_single_process_step(world):
    E, R, h, r, y = _problem()
    E1, R1, l1 = ps.reference_step(E, R, h, r, y, lr=0.7)
    E2, R2, l2 = ps.run_sharded_step(world, E, R, h, r, y, lr=0.7)
    assert np.allclose(E1, E2, atol=1e-12) and np.allclose(R1, R2, atol=1e-12) and abs(l1 - l2) < 1e-12


def test_two_steps_match_and_the_closing_barrier_orders_the_next_lookup():
    E, R, h, r, y = _problem(seed=1)
    Ea, Ra, _ = ps.reference_step(E, R, h, r, y, lr=0.3)
    Ea, Ra, la = ps.reference_step(Ea, Ra, h, r, y, lr=0.3)
    Eb, Rb, lb = ps.run_sharded_step(3, E, R, h, r, y, lr=0.3, steps=2)
    assert np.allclose(Ea, Eb, atol=1e-12) and np.allclose(Ra, Rb, atol=1e-12) and abs(la - lb) < 1e-12
    with pytest.raises(ps.ProtocolHazard):
        ps.run_sharded_step(3, E, R, h, r, y, lr=0.3, steps=2, skip_barrier="S3")


@pytest.mark.parametrize("name", ["S1", "S2", "S2b", "S3"])
def test_removed_barrier_is_reported_as_hazard(name):
    E, R, h, r, y = _problem(seed=2)
    with pytest.raises(ps.ProtocolHazard):
        ps.run_sharded_step(4, E, R, h, r, y, lr=0.1, skip_barrier=name)


def test_absent_rank_ends_in_bounded_timeout():
    E, R, h, r, y = _problem(seed=3)
    with pytest.raises(ps.PeerTimeout) as ei:
        ps.run_sharded_step(3, E, R, h, r, y, lr=0.1, absent_rank=2, poll_limit=200)
    assert ei.value.missing == [2]


def test_dropped_signal_ends_in_bounded_timeout():
    E, R, h, r, y = _problem(seed=4)
    drop = lambda sender, peer, count: sender == 0 and peer == 1 and count == 2   # noqa: E731 - S2's signal 0 -> 1
    with pytest.raises(ps.PeerTimeout) as ei:
        ps.run_sharded_step(2, E, R, h, r, y, lr=0.1, drop=drop, poll_limit=300)
    assert ei.value.rank == 1 and ei.value.missing == [0]


def test_barrier_counter_semantics():
    b = ps.SimBarrier(2, poll_limit=5, poll_sleep=0.0)
    assert b.arrive_and_wait(0) == ps.ST_TIMEOUT_PEER and b.missing(0) == [1]
    assert b.arrive_and_wait(1) == ps.ST_OK          # rank 0's signal is already there


def test_heartbeat_detects_silent_rank():
    store, now = DictStore(), [0.0]
    hb = [Heartbeat(store, k, 3, timeout=5.0, clock=lambda: now[0]) for k in range(3)]
    for t in range(4):
        now[0] = float(t)
        for k in range(3):
            hb[k].beat()
        hb[0].check()
    for t in range(4, 12):                              # rank 2 stops beating
        now[0] = float(t)
        hb[0].beat(); hb[1].beat()
        if t < 9:
            hb[0].check()
    with pytest.raises(RankFailure) as ei:
        hb[0].check()
    assert ei.value.rank == 2
    with pytest.raises(RankFailure):                    # sticky until the job is restarted
        hb[0].raise_if_failed()


def test_heartbeat_background_thread():
    import time
    store = DictStore()
    a = Heartbeat(store, 0, 2, timeout=0.3, interval=0.05).start()
    b = Heartbeat(store, 1, 2, timeout=0.3, interval=0.05).start()
    time.sleep(0.3)
    a.raise_if_failed(); b.raise_if_failed()
    b.stop()                                            # rank 1 goes away between steps
    deadline = time.time() + 5
    while a.failure is None and time.time() < deadline:
        time.sleep(0.05)
    a.stop()
    assert isinstance(a.failure, RankFailure) and a.failure.rank == 1
