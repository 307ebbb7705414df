"""CPU model of the exchange protocol: dropped, late, duplicate and reordered deliveries."""

import random

from lplb_b200.parallel.protocol_model import Fabric, Rank, run_lockstep, two_level_step


def _truth(counts, n_elems):
    return [sum(c[e] for c in counts) for e in range(n_elems)]


def test_lockstep_sums_are_exact_for_every_rank():
    for n_ranks in (2, 4, 8):
        for counts, results in run_lockstep(n_ranks, 16, steps=7, seed=n_ranks):
            want = _truth(counts, 16)
            for sums, miss in results:
                assert miss == 0 and sums == want


def test_fast_rank_one_launch_ahead_never_corrupts_a_slow_reader():
    # rank 0 publishes epoch n+1 before rank 1 has read epoch n: different parity, no overlap;
    # rank 0 cannot publish epoch n+2 because it never finished n+1 without rank 1's words.
    n, e = 2, 8
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    c0, c1 = [1] * e, [10] * e
    ranks[0].publish(c0, fab)
    ranks[1].publish(c1, fab)
    fab.deliver_all(ranks)
    assert ranks[0].finish() == ([11] * e, 0)
    # rank 0 races ahead into epoch 2 while rank 1 has not summed epoch 1 yet
    ranks[0].publish([2] * e, fab)
    fab.deliver_all(ranks)
    assert ranks[1].finish() == ([11] * e, 0)  # epoch-1 buffer untouched
    assert ranks[0].ready() == [True, False]  # rank 0 is stuck in epoch 2 until rank 1 arrives
    ranks[1].publish([20] * e, fab)
    fab.deliver_all(ranks)
    assert ranks[0].finish() == ([22] * e, 0) and ranks[1].finish() == ([22] * e, 0)


def test_partial_delivery_is_not_mistaken_for_arrival():
    n, e = 2, 4
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    ranks[0].publish([5, 6, 7, 8], fab)
    ranks[1].publish([1, 1, 1, 1], fab)
    # deliver everything except one word of rank 1 -> rank 0
    for key in fab.pending():
        if key[:2] == (1, 0) and key[3] == 2:
            continue
        fab.deliver(key, ranks)
    assert ranks[0].ready() == [True, False]
    sums, miss = ranks[0].finish()  # budget ran out: rank 1 is reported, own counts stand in
    assert miss == 0b10 and sums == [10, 12, 14, 16]
    assert ranks[1].finish() == ([6, 7, 8, 9], 0)


def test_dropped_rank_times_out_everywhere_and_late_words_are_ignored_later():
    n, e = 4, 4
    rng = random.Random(3)
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    counts = [[r + 1] * e for r in range(n)]
    # epoch 1: rank 3's stores are held back (it is slow), everyone else times out on it
    for r in ranks:
        r.publish(counts[r.rank], fab)
    held = [k for k in fab.pending() if k[0] == 3 and k[1] != 3]
    for key in fab.pending():
        if key not in held:
            fab.deliver(key, ranks)
    for r in ranks[:3]:
        sums, miss = r.finish()
        assert miss == 0b1000
        assert sums == [1 + 2 + 3 + (r.rank + 1)] * e  # own counts replace rank 3's
    # epochs 2 and 3 run normally; the held epoch-1 words land in the middle of epoch 3,
    # whose parity they share, *before* rank 3's epoch-3 words (same-address FIFO)
    for _ in range(2):
        for r in ranks:
            r.publish(counts[r.rank], fab)
        if ranks[0].epoch == 2:  # other parity: the held words stay in flight
            for key in [k for k in fab.pending() if k not in held]:
                fab.deliver(key, ranks)
        else:
            for key in held:  # pops the epoch-1 word, the epoch-3 word queues behind it
                fab.deliver(key, ranks)
            assert ranks[0].ready()[3] is False  # tag 1 is not tag 3
            fab.deliver_all(ranks, rng)
        for r in ranks:
            assert r.finish() == ([10] * e, 0)


def test_duplicate_delivery_is_harmless():
    n, e = 2, 3
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    ranks[0].publish([1, 2, 3], fab)
    ranks[1].publish([4, 5, 6], fab)
    for key in fab.pending():
        fab.deliver(key, ranks, duplicate=True)
    fab.deliver_all(ranks)
    assert ranks[0].finish() == ([5, 7, 9], 0) and ranks[1].finish() == ([5, 7, 9], 0)


def test_reset_realigns_epochs_after_a_skipped_launch():
    # rank 1 skips a launch: its epoch falls behind, every later exchange would time out
    n, e = 2, 2
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    ranks[0].publish([1, 1], fab)
    fab.deliver_all(ranks)
    assert ranks[0].finish()[1] == 0b10
    ranks[0].publish([1, 1], fab)
    ranks[1].publish([2, 2], fab)  # epoch 1 on rank 1, epoch 2 on rank 0
    fab.deliver_all(ranks)
    # the rank that is ahead keeps timing out (that is how the host learns about it); the
    # lagging rank meanwhile reads the leader's *previous* words, whose tag equals its epoch
    assert ranks[0].finish()[1] == 0b10
    assert ranks[1].finish() == ([3, 3], 0)
    # the host-side reset (Planner.reset_exchange) zeroes epochs and buffers on every rank
    ranks = [Rank(r, n, e) for r in range(n)]
    ranks[0].publish([1, 1], fab)
    ranks[1].publish([2, 2], fab)
    fab.deliver_all(ranks)
    assert ranks[0].finish() == ([3, 3], 0) and ranks[1].finish() == ([3, 3], 0)


def test_two_level_schedule_gives_every_rank_the_global_sum():
    rng = random.Random(5)
    for n, node in ((4, 2), (8, 4), (8, 2)):
        e = 6
        ranks = [Rank(r, n, e) for r in range(n)]
        fab = Fabric(n, e)
        for _ in range(5):  # several launches: both parities, both levels reused
            counts = [[rng.randrange(1 << 16) for _ in range(e)] for _ in range(n)]
            want = _truth(counts, e)
            for sums, miss in two_level_step(ranks, fab, counts, node, lambda level: fab.deliver_all(ranks, rng)):
                assert miss == 0 and sums == want


def test_two_level_levels_do_not_share_slots():
    # A level-1 word from a rank must not satisfy (or overwrite) the level-0 wait on that rank.
    n, node, e = 4, 2, 3
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    counts = [[r + 1] * e for r in range(n)]
    two_level_step(ranks, fab, counts, node)
    # own level-1 word sits in slot [1][level 1][0]; the level-0 slot of the same source holds the raw counts
    assert [w & 0xFFFFFFFF for w in ranks[0].recv[1][0][0]] == [1] * e
    assert [w & 0xFFFFFFFF for w in ranks[0].recv[1][1][0]] == [3] * e  # node sum of ranks 0 and 1
    assert [w & 0xFFFFFFFF for w in ranks[0].recv[1][1][2]] == [7] * e  # node sum of ranks 2 and 3


def test_two_level_late_rank_is_reported_in_every_node():
    # Rank 3's level-0 words to its node peer (rank 2) are held back.  Rank 2 reports it,
    # substitutes its own counts and marks its node sum as degraded, so its partner in the
    # other node (rank 0) reports rank 2's vector too.  Rank 3's own node sum was complete,
    # so ranks 1 and 3 end with the true total and no report: totals can differ between
    # ranks after a timeout, but no rank uses a substituted share without saying so.
    n, node, e = 4, 2, 2
    ranks = [Rank(r, n, e) for r in range(n)]
    fab = Fabric(n, e)
    counts = [[1] * e, [2] * e, [4] * e, [8] * e]

    def deliver(level):
        for key in fab.pending():
            if level == 0 and key[0] == 3 and key[1] == 2:
                continue
            while fab.queues[key]:
                fab.deliver(key, ranks)

    res = two_level_step(ranks, fab, counts, node, deliver)
    assert res[2] == ([1 + 2 + 4 + 4] * e, 0b1100)   # saw the timeout itself (bit 3) and its own degraded word (bit 2)
    assert res[0] == ([1 + 2 + 4 + 4] * e, 0b0100)   # partner of rank 2: told by the degraded mark
    assert res[1] == ([1 + 2 + 4 + 8] * e, 0)        # partner of rank 3, whose own node sum was complete
    assert res[3] == ([1 + 2 + 4 + 8] * e, 0)
