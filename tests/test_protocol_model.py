"""Safety properties of the cross-rank flag protocol, checked on a host model (threads = thread blocks)."""
import threading

import pytest

from apexw_b200.parallel import protocol_model as pm


def test_epoch_comparison_wraps():
    assert pm.reached(5, 5) and pm.reached(6, 5) and not pm.reached(4, 5)
    assert pm.reached(2, 0xFFFFFFFE)            # 2 is four launches after 0xFFFFFFFE
    assert not pm.reached(0xFFFFFFFE, 2)


@pytest.mark.parametrize("world,blocks", [(2, 3), (4, 2), (8, 2)])
def test_no_block_works_before_every_rank_arrived_and_no_rank_leaves_before_all_wrote(world, blocks):
    w = pm.World(world)
    lock = threading.Lock()
    arrived, wrote, violations = set(), [], []

    for epoch in (1, 2, 3):
        arrived.clear()
        wrote.clear()

        def body(rank, block, epoch=epoch):
            # entry property: every rank's entry flag for this epoch is visible in this rank's pad
            for r in range(world):
                if not pm.reached(w.load(rank, r), epoch):
                    violations.append(("entry", rank, r))
            with lock:
                wrote.append(rank)

        pm.run_launch(w, epoch, blocks, 2.0, body, delays={world - 1: 0.05})
        assert not violations
        assert sorted(wrote) == sorted(list(range(world)) * blocks)
        assert w.status == [pm.OK] * world
        # exit property: when a rank's launch has ended, every peer's exit flag for the epoch is in its pad
        for rank in range(world):
            assert all(pm.reached(w.load(rank, pm.MAX_PEERS + r), epoch) for r in range(world))
            assert w.load(rank, pm.DONE) == 0


def test_missing_rank_times_out_everywhere_and_nobody_runs_the_body():
    w = pm.World(3)
    ran = []
    pm.run_launch(w, 1, 2, 0.05, lambda r, b: ran.append(r), ranks=[0, 1])     # rank 2 never launches
    assert ran == []
    assert w.status[0] == pm.ENTRY_TIMEOUT and w.status[1] == pm.ENTRY_TIMEOUT
    # the abort verdict of epoch 1 must not be mistaken for the go word of epoch 2
    assert not pm.reached(w.load(0, pm.GO), 2) or w.load(0, pm.GO) != 2


def test_stale_flags_of_an_earlier_epoch_do_not_release_the_next_launch():
    w = pm.World(2)
    pm.run_launch(w, 1, 1, 1.0, lambda r, b: None)
    ran = []
    pm.run_launch(w, 2, 1, 0.05, lambda r, b: ran.append(r), ranks=[0])         # rank 1 is a launch behind
    assert ran == [] and w.status[0] == pm.ENTRY_TIMEOUT


def test_late_rank_is_waited_for_within_the_budget():
    w = pm.World(2)
    ran = []
    pm.run_launch(w, 7, 2, 2.0, lambda r, b: ran.append(r), delays={1: 0.2})
    assert sorted(ran) == [0, 0, 1, 1] and w.status == [pm.OK, pm.OK]


# ---- the partial-sum exchange of a clipped step (zero_norm_exchange_kernel) ------------------------------------

def _clipped_steps(world, steps, values, delays=None, blocks=2, budget_s=2.0, missing=()):
    """Every step: exchange of the partial sums, then one update launch (entry round, body, exit round), as the
    optimizer issues them; epochs advance by one per launch.  Returns totals[step][rank] and the world."""
    import threading
    import time
    from apexw_b200.parallel import protocol_model as pm

    w = pm.World(world)
    totals = [[None] * world for _ in range(steps)]
    delays = delays or {}

    def rank_fn(rank):
        epoch = 0
        for s in range(steps):
            time.sleep(delays.get((s, rank), 0.0))
            epoch += 1
            totals[s][rank] = pm.norm_exchange(w, rank, epoch, values[s][rank], budget_s)
            epoch += 1
            # the update launch of this rank: `blocks` thread blocks, run here one after the other's start
            ts = [threading.Thread(target=lambda b=b, e=epoch: (pm.peer_entry(w, rank, b, e, budget_s)
                                                                 and pm.peer_exit(w, rank, blocks, e, budget_s)))
                  for b in range(blocks)]
            for t in ts:
                t.start()
            for t in ts:
                t.join()

    threads = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world) if r not in missing]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return totals, w


@pytest.mark.parametrize("world", [2, 4, 8])
def test_every_rank_gets_the_same_total_in_rank_order(world):
    from apexw_b200.parallel import protocol_model as pm
    values = [[(s + 1) * 0.1 + r * 1e-3 for r in range(world)] for s in range(3)]
    totals, w = _clipped_steps(world, 3, values)
    for s in range(3):
        want = 0.0
        for v in values[s]:
            want += v                      # the same left-to-right sum on every rank: bit-identical totals
        assert all(t == (want, True) for t in totals[s]), (s, totals[s])
    assert w.status == [pm.OK] * world


def test_a_slow_rank_never_makes_the_others_read_last_steps_sum():
    """Rank 1 arrives late in step 2: its slot still holds step 1's value, but its flag holds step 1's epoch, so the
    others wait instead of reading the stale number."""
    values = [[1.0, 2.0, 4.0], [10.0, 20.0, 40.0], [100.0, 200.0, 400.0]]
    totals, _ = _clipped_steps(3, 3, values, delays={(1, 1): 0.15, (2, 0): 0.1})
    assert [t[0] for t in totals[0]] == [7.0] * 3
    assert [t[0] for t in totals[1]] == [70.0] * 3
    assert [t[0] for t in totals[2]] == [700.0] * 3


def test_the_value_is_in_place_before_its_flag_can_be_seen():
    """Value first, flag second: a reader that sees the flag sees the value, however long the writer dawdles between
    the two stores."""
    import threading
    import time
    from apexw_b200.parallel import protocol_model as pm
    w = pm.World(2)
    out = {}

    def slow_writer():
        out[0] = pm.norm_exchange(w, 0, 1, 3.0, 2.0, between=lambda r: time.sleep(0.05))

    def reader():
        out[1] = pm.norm_exchange(w, 1, 1, 5.0, 2.0)

    ts = [threading.Thread(target=slow_writer), threading.Thread(target=reader)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert out[0] == (8.0, True) and out[1] == (8.0, True)


def test_a_missing_rank_ends_the_exchange_with_a_status_and_no_clipping():
    from apexw_b200.parallel import protocol_model as pm
    values = [[1.0, 2.0, 4.0]]
    totals, w = _clipped_steps(3, 1, values, budget_s=0.1, missing=(2,))
    assert totals[0][0] == (0.0, False) and totals[0][1] == (0.0, False)
    assert w.status[0] == pm.ENTRY_TIMEOUT and w.status[1] == pm.ENTRY_TIMEOUT
