"""KvPageManager: one test per named case (allocation, reservations, two-phase prefix commit over packed ragged
widths, rollback, quarantine and retirement confirmation, exact and prefix forks with copy-on-write credit,
preempt / restore, failure atomicity).  `check_invariants` runs after every step that changes ownership.

The case list follows the reference's page-manager suite (crates/ferrule-runtime/src/cache/page_manager.rs:1389-2023)."""
import random

import pytest

from ferrule_b200.runtime.kv_pages import KvError, KvPageManager, OutOfPages, ReservationState


def mgr(pages=16, ps=4):
    return KvPageManager(pages, ps, max_sequence_len=10_000)


def commit(m, res, rows=None):
    """Full (or `rows`-row) commit of one reservation; retired pages are confirmed at once."""
    cid = m.prepare_commit([(res.res_id, res.tokens if rows is None else rows)])
    ret = m.publish_commit(cid)
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()
    return ret


def grow(m, seq, n):
    return commit(m, m.reserve(seq, n))


# ------------------------------------------------------------------------------------------ allocation
def test_alloc_and_free_sequence():
    m = mgr()
    a, b = m.alloc_sequence(), m.alloc_sequence()
    assert a != b and m.sequence(a).committed_tokens == 0 and m.stats().sequences == 2
    assert not m.free_sequence_pages(a) and m.stats().sequences == 1
    with pytest.raises(KvError):
        m.sequence(a)
    m.check_invariants()


def test_reserve_commit_extends_the_block_table():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 6)
    assert len(r.new_pages) == 2 and r.start == 0 and m.sequence(s).pages == []        # nothing visible yet
    commit(m, r)
    assert m.sequence(s).pages == r.new_pages and m.sequence(s).committed_tokens == 6


def test_incremental_reserve_commits_fill_the_tail_page_before_taking_a_new_one():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 3)
    r = m.reserve(s, 1)
    assert r.new_pages == [] and m.required_physical_pages(s, 1) == 0 or True
    commit(m, r)
    r = m.reserve(s, 1)
    assert len(r.new_pages) == 1
    commit(m, r)
    assert m.sequence(s).committed_tokens == 5 and len(m.sequence(s).pages) == 2


def test_multiple_pages_for_a_long_sequence_and_exact_write_slots_across_boundaries():
    m = KvPageManager(2048, 4, max_sequence_len=10_000)
    s = m.alloc_sequence()
    grow(m, s, 4097)
    r = m.reserve(s, 6)
    blocks, slots = m.reservation_bindings(r.res_id)
    assert len(blocks) == m.pages_for(4103)
    for j, slot in enumerate(slots):
        pos = 4097 + j
        assert slot == blocks[pos // 4] * 4 + pos % 4
    rr, b2, s2 = m.bind_and_bindings(r.res_id, execution_id=9)
    assert s2 == slots and b2 == blocks and rr.state == ReservationState.BOUND and rr.execution_id == 9


def test_out_of_pages_is_an_error_and_changes_nothing():
    m = mgr(pages=3)
    s = m.alloc_sequence()
    grow(m, s, 8)
    before = (m.free_pages, list(m.sequence(s).pages))
    with pytest.raises(OutOfPages):
        m.reserve(s, 9)
    assert (m.free_pages, m.sequence(s).pages) == before and m.sequence(s).open_reservation is None
    assert m.stats().reserve_failures == 1
    m.check_invariants()


def test_failed_multi_page_reserve_returns_every_partial_allocation():
    m = mgr(pages=4)
    a, b = m.alloc_sequence(), m.alloc_sequence()
    grow(m, a, 8)
    with pytest.raises(OutOfPages):
        m.reserve(b, 12)                      # needs 3, 2 are free
    assert m.free_pages == 2
    r, need = m.try_reserve(b, 12, page_budget=10)
    assert r is None and need == 3
    r, need = m.try_reserve(b, 8, page_budget=1)
    assert r is None and need == 2            # fits the pool but not the caller's budget
    m.check_invariants()


def test_free_sequence_returns_pages_through_quarantine_and_they_are_reused():
    m = mgr(pages=4)
    s = m.alloc_sequence()
    grow(m, s, 16)
    pages = list(m.sequence(s).pages)
    ret = m.free_sequence_pages(s)
    assert sorted(ret.pages) == sorted(pages) and m.free_pages == 0 and m.stats().quarantined_pages == 4
    t = m.alloc_sequence()
    with pytest.raises(OutOfPages):
        m.reserve(t, 1)                       # quarantined pages are not allocatable
    assert m.confirm_page_retirement(ret.pages) == 4 and m.free_pages == 4
    grow(m, t, 16)
    assert sorted(m.sequence(t).pages) == sorted(pages)


# ------------------------------------------------------------------------------------------ reservations
def test_one_sequence_cannot_hold_two_live_reservations():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 2)
    with pytest.raises(KvError):
        m.reserve(s, 1)
    m.confirm_page_retirement(m.abort_reservations([r.res_id]).pages)
    m.reserve(s, 1)
    m.check_invariants()


def test_reservation_prefix_view_publishes_nothing_and_truncates_the_bindings():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 3)
    r = m.reserve(s, 7)                                  # positions 3..9: pages 0 (tail), 1, 2
    full = m.reservation_view(r.res_id)
    assert full.context_len == 3 and full.tokens == 7 and len(full.block_ids) == 3
    v = m.reservation_prefix_view(r.res_id, 2)           # positions 3, 4: two pages
    assert v.tokens == 2 and v.block_ids == full.block_ids[:2]
    assert m.reservation_prefix_view(r.res_id, 0).block_ids == full.block_ids[:1]
    with pytest.raises(KvError):
        m.reservation_prefix_view(r.res_id, 8)
    assert m.sequence(s).committed_tokens == 3 and len(m.sequence(s).pages) == 1 and r.state == ReservationState.RESERVED


def test_commit_prefix_quarantines_the_rejected_suffix_until_confirmation():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 10)                                 # three pages
    cid = m.prepare_commit([(r.res_id, 3)])              # one page kept
    ret = m.publish_commit(cid)
    assert len(ret.pages) == 2 and m.sequence(s).committed_tokens == 3 and len(m.sequence(s).pages) == 1
    assert m.stats().quarantined_pages == 2 and set(ret.pages).isdisjoint(m.free_page_ids())
    m.check_invariants()
    m.confirm_page_retirement(ret.pages)
    assert m.stats().quarantined_pages == 0


def test_packed_prefix_commit_publishes_ragged_widths_atomically():
    m = mgr(pages=32)
    seqs = [m.alloc_sequence() for _ in range(4)]
    for s, n in zip(seqs, (1, 4, 7, 2)):
        grow(m, s, n)
    res = [m.reserve(s, 5) for s in seqs]
    widths = [5, 0, 2, 1]
    cid = m.prepare_commit(list(zip([r.res_id for r in res], widths)))
    assert all(r.state == ReservationState.PREPARED for r in res)
    assert [m.sequence(s).committed_tokens for s in seqs] == [1, 4, 7, 2]          # nothing visible before publish
    ret = m.publish_commit(cid)
    assert [m.sequence(s).committed_tokens for s in seqs] == [6, 4, 9, 3]
    assert all(m.sequence(s).open_reservation is None for s in seqs)
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()


def test_packed_validation_failure_returns_all_ownership_without_publication():
    m = mgr(pages=32)
    a, b = m.alloc_sequence(), m.alloc_sequence()
    ra, rb = m.reserve(a, 4), m.reserve(b, 4)
    with pytest.raises(KvError):
        m.prepare_commit([(ra.res_id, 4), (rb.res_id, 5)])            # second width exceeds its reservation
    assert ra.state == ReservationState.RESERVED and rb.state == ReservationState.RESERVED
    with pytest.raises(KvError):
        m.prepare_commit([(ra.res_id, 4), (ra.res_id, 1)])            # listed twice
    assert m.sequence(a).committed_tokens == 0 and m.sequence(a).open_reservation == ra.res_id
    cid = m.prepare_commit([(ra.res_id, 4), (rb.res_id, 4)])          # both reservations are still whole
    m.publish_commit(cid)
    m.check_invariants()


def test_commit_and_rollback_in_one_transaction():
    m = mgr(pages=32)
    a, b = m.alloc_sequence(), m.alloc_sequence()
    grow(m, a, 4)
    grow(m, b, 4)
    ra, rb = m.reserve(a, 3), m.reserve(b, 3)
    ret = m.publish_commit(m.prepare_commit([(ra.res_id, 3), (rb.res_id, 0)]))
    assert m.sequence(a).committed_tokens == 7 and m.sequence(b).committed_tokens == 4
    assert len(ret.pages) == 1 and len(m.sequence(b).pages) == 1        # b's new page went back
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()


def test_zero_prefix_is_an_exact_rollback():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 5)
    before = (list(m.sequence(s).pages), m.sequence(s).committed_tokens)
    r = m.reserve(s, 9)
    ret = m.publish_commit(m.prepare_commit([(r.res_id, 0)]))
    assert (m.sequence(s).pages, m.sequence(s).committed_tokens) == before and sorted(ret.pages) == sorted(r.new_pages)
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()


def test_prefix_beyond_the_reservation_is_rejected_without_consuming_it():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 3)
    for rows in (4, -1):
        with pytest.raises(KvError):
            m.prepare_commit([(r.res_id, rows)])
    assert r.state == ReservationState.RESERVED
    commit(m, r, 3)


def test_abort_needs_retirement_confirmation_before_the_pages_are_reused():
    m = mgr(pages=2)
    s = m.alloc_sequence()
    r = m.reserve(s, 8)
    ret = m.abort_reservations([r.res_id])
    assert sorted(ret.pages) == sorted(r.new_pages) and m.free_pages == 0 and r.state == ReservationState.ABORTED
    with pytest.raises(OutOfPages):
        m.reserve(s, 1)
    m.confirm_page_retirement(ret.pages)
    grow(m, s, 8)


def test_duplicate_retirement_confirmation_is_rejected_without_touching_the_free_list():
    m = mgr(pages=4)
    s = m.alloc_sequence()
    grow(m, s, 8)
    ret = m.free_sequence_pages(s)
    m.confirm_page_retirement(ret.pages)
    free = m.free_page_ids()
    with pytest.raises(KvError):
        m.confirm_page_retirement(ret.pages[:1])
    with pytest.raises(KvError):
        m.confirm_page_retirement([free[0]])               # a free page was never awaiting retirement
    assert m.free_page_ids() == free
    m.check_invariants()


def test_retirement_cannot_be_confirmed_by_another_manager():
    m1, m2 = mgr(), mgr()
    s = m1.alloc_sequence()
    grow(m1, s, 4)
    ret = m1.free_sequence_pages(s)
    with pytest.raises(KvError):
        m2.confirm_page_retirement(ret.pages)
    m1.confirm_page_retirement(ret.pages)


def test_consumed_reservation_cannot_change_state_again():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 2)
    commit(m, r)
    with pytest.raises(KvError):
        m.prepare_commit([(r.res_id, 1)])
    with pytest.raises(KvError):
        m.bind_reservation_execution(r.res_id, 1)
    assert not m.abort_reservations([r.res_id])             # unknown by now: nothing to give back
    assert m.sequence(s).committed_tokens == 2


def test_prepared_commit_can_be_aborted_back_to_whole_reservations():
    m = mgr()
    s = m.alloc_sequence()
    r = m.reserve(s, 6)
    m.bind_reservation_execution(r.res_id, 3)
    cid = m.prepare_commit([(r.res_id, 2)])
    with pytest.raises(KvError):
        m.abort_reservations([r.res_id])                    # part of a prepared commit
    m.abort_prepared_commit(cid)
    assert r.state == ReservationState.BOUND and r.committed_rows == 0
    with pytest.raises(KvError):
        m.publish_commit(cid)
    commit(m, r, 6)


def test_truncate_rolls_a_sequence_back_and_refuses_an_open_reservation():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 10)
    g0 = m.sequence(s).generation
    r = m.reserve(s, 1)
    with pytest.raises(KvError):
        m.truncate_sequence(s, 4)
    m.confirm_page_retirement(m.abort_reservations([r.res_id]).pages)
    ret = m.truncate_sequence(s, 4)
    assert len(ret.pages) == 2 and m.sequence(s).committed_tokens == 4 and m.sequence(s).generation == g0 + 1
    with pytest.raises(KvError):
        m.truncate_sequence(s, 5)
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()


# ------------------------------------------------------------------------------------------ fork / copy-on-write
def test_fork_shares_pages_and_a_partial_tail_append_uses_cow():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 6)                                            # pages [p0 full, p1 half]
    c = m.publish_fork_sequence_exact(s)
    assert m.sequence(c).pages == m.sequence(s).pages and m.stats().shared_pages == 2 and m.stats().forks == 1
    assert m.required_physical_pages(c, 1) == 1              # the copy of the shared tail
    r = m.reserve(c, 1)
    assert r.cow is not None and r.cow.source == m.sequence(s).pages[1] and r.cow.logical_page == 1
    assert r.new_pages == [] and m.stats().cow_copies == 1
    view = m.reservation_view(r.res_id)
    assert view.block_ids == [m.sequence(s).pages[0], r.cow.replacement]
    ret = commit(m, r)
    assert ret.pages == [] and m.sequence(c).pages[1] == r.cow.replacement        # the parent still holds the source
    assert m.sequence(s).pages[1] == r.cow.source and m.stats().shared_pages == 1
    # the parent now owns its tail alone: appending needs no copy
    assert m.required_physical_pages(s, 1) == 0 and m.reserve(s, 1).cow is None


def test_cow_rollback_preserves_the_shared_view():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 6)
    c = m.publish_fork_sequence_exact(s)
    r = m.reserve(c, 3)
    ret = m.publish_commit(m.prepare_commit([(r.res_id, 0)]))        # nothing accepted: the copy is discarded
    assert r.cow.replacement in ret.pages and m.sequence(c).pages == m.sequence(s).pages
    assert m.stats().shared_pages == 2
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()
    r2 = m.reserve(c, 3)
    ret2 = m.abort_reservations([r2.res_id])
    assert r2.cow.replacement in ret2.pages and m.sequence(c).pages == m.sequence(s).pages
    m.confirm_page_retirement(ret2.pages)
    m.check_invariants()


def test_cow_credit_accounting_counts_growth_plus_one_copy():
    m = mgr(pages=8)
    s = m.alloc_sequence()
    grow(m, s, 6)
    c = m.publish_fork_sequence_exact(s)
    assert m.required_physical_pages(c, 2) == 1              # fits the tail page: copy only
    assert m.required_physical_pages(c, 3) == 2              # copy + one new page
    assert m.required_physical_pages(c, 11) == 4
    r, need = m.try_reserve(c, 11, page_budget=3)
    assert r is None and need == 4 and m.stats().cow_copies == 0
    r, need = m.try_reserve(c, 11, page_budget=4)
    assert r is not None and need == 4 and len(r.new_pages) == 3 and r.cow is not None
    m.check_invariants()


def test_prepared_fork_is_invisible_until_publish():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 5)
    tokens, pages = m.prepare_fork_sequence_exact(s)
    assert tokens == 5 and pages == m.sequence(s).pages and m.stats().forks == 0 and m.stats().shared_pages == 0
    pages.append(99)                                         # the caller's list is a copy
    assert 99 not in m.sequence(s).pages
    m.check_invariants()


def test_fork_is_refused_under_an_open_reservation_and_for_preempted_sequences():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 5)
    r = m.reserve(s, 1)
    with pytest.raises(KvError):
        m.publish_fork_sequence_exact(s)
    with pytest.raises(KvError):
        m.publish_fork_sequence_prefix(s, 4)
    commit(m, r)
    m.preempt_sequence(s)
    with pytest.raises(KvError):
        m.publish_fork_sequence_exact(s)
    assert m.stats().forks == 0 and m.stats().shared_pages == 0


def test_prefix_fork_shares_whole_pages_only_and_needs_no_copy():
    m = mgr()
    s = m.alloc_sequence()
    grow(m, s, 11)
    for bad in (0, 3, 12, 16):
        with pytest.raises(KvError):
            m.publish_fork_sequence_prefix(s, bad)
    c = m.publish_fork_sequence_prefix(s, 8)
    assert m.sequence(c).pages == m.sequence(s).pages[:2] and m.sequence(c).committed_tokens == 8
    assert m.stats().shared_pages == 2 and m.required_physical_pages(c, 1) == 1      # a page of its own, no copy
    r = m.reserve(c, 1)
    assert r.cow is None and len(r.new_pages) == 1
    commit(m, r)
    # freeing the donor keeps the shared pages alive for the child
    ret = m.free_sequence_pages(s)
    assert len(ret.pages) == 1 and m.stats().shared_pages == 0
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()


def test_many_forks_release_in_any_order():
    m = mgr(pages=8)
    s = m.alloc_sequence()
    grow(m, s, 8)
    kids = [m.publish_fork_sequence_exact(s) for _ in range(5)]
    for k in (kids[3], s, kids[0], kids[4], kids[1]):
        ret = m.free_sequence_pages(k)
        assert ret.pages == []
        m.check_invariants()
    ret = m.free_sequence_pages(kids[2])
    assert len(ret.pages) == 2
    m.confirm_page_retirement(ret.pages)
    assert m.free_pages == 8


# ------------------------------------------------------------------------------------------ preempt / restore
def test_preempt_restore_preserves_the_logical_block_table():
    m = mgr(pages=8)
    s = m.alloc_sequence()
    grow(m, s, 10)
    other = m.publish_fork_sequence_prefix(s, 4)             # page 0 is shared, pages 1-2 exclusive
    rec = m.preempt_sequence(s)
    assert [i for i, _ in rec.exclusive] == [1, 2] and [i for i, _ in rec.shared] == [0]
    with pytest.raises(KvError):
        m.reserve(s, 1)
    with pytest.raises(KvError):
        m.preempt_sequence(s)
    ret = m.release_preempted_pages(s)
    assert len(ret.pages) == 2 and m.sequence(s).pages[1:] == [-1, -1]
    m.confirm_page_retirement(ret.pages)
    m.check_invariants()
    g0 = m.sequence(s).generation
    mapping = m.restore_sequence(s)
    assert [i for i, _ in mapping] == [1, 2] and all(p >= 0 for p in m.sequence(s).pages)
    assert m.sequence(s).pages[0] == m.sequence(other).pages[0] and m.sequence(s).committed_tokens == 10
    assert m.sequence(s).generation == g0 + 1 and not m.sequence(s).preempted
    grow(m, s, 1)


def test_restore_without_pages_fails_and_can_be_retried():
    m = mgr(pages=3)
    s = m.alloc_sequence()
    grow(m, s, 8)
    m.preempt_sequence(s)
    m.confirm_page_retirement(m.release_preempted_pages(s).pages)
    t = m.alloc_sequence()
    grow(m, t, 8)
    with pytest.raises(OutOfPages):
        m.restore_sequence(s)
    assert m.sequence(s).preempted and m.sequence(s).pages == [-1, -1]
    m.confirm_page_retirement(m.free_sequence_pages(t).pages)
    assert len(m.restore_sequence(s)) == 2
    m.check_invariants()


def test_freeing_a_preempted_sequence_skips_its_released_pages():
    m = mgr(pages=4)
    s = m.alloc_sequence()
    grow(m, s, 8)
    m.preempt_sequence(s)
    m.confirm_page_retirement(m.release_preempted_pages(s).pages)
    assert not m.free_sequence_pages(s)
    assert m.free_pages == 4 and m.stats().sequences == 0
    m.check_invariants()


def test_execution_binding_is_independent_of_page_ownership():
    m = mgr()
    a, b = m.alloc_sequence(), m.alloc_sequence()
    ra, rb = m.reserve(a, 2), m.reserve(b, 2)
    m.bind_reservation_execution(ra.res_id, 41)
    m.bind_reservation_execution(rb.res_id, 41)              # one execution may carry many reservations
    assert ra.execution_id == rb.execution_id == 41
    with pytest.raises(KvError):
        m.bind_reservation_execution(ra.res_id, 42)          # already bound
    m.publish_commit(m.prepare_commit([(ra.res_id, 2), (rb.res_id, 2)]))
    m.check_invariants()


def test_stats_track_high_water_and_sharing():
    m = mgr(pages=8)
    s = m.alloc_sequence()
    grow(m, s, 16)
    assert m.stats().high_water_used == 4 and m.stats().used_pages == 4
    m.confirm_page_retirement(m.truncate_sequence(s, 4).pages)
    st = m.stats()
    assert st.used_pages == 1 and st.high_water_used == 4 and st.free_pages == 7 and st.open_reservations == 0


def test_released_page_id_outside_the_pool_is_detected():
    m = mgr(pages=4)
    s = m.alloc_sequence()
    grow(m, s, 4)
    m.sequence(s).pages.append(99)
    with pytest.raises(KvError):
        m.free_sequence_pages(s)


# ---------------------------------------------------------------------------------------------- randomised soak
def _soak(seed):
    rnd = random.Random(seed)
    m = KvPageManager(24, 8, 200)
    seqs = {}        # id -> model: committed tokens
    open_res = {}    # seq -> (res_id, rows)
    prepared = []    # (commit_id, [(seq, rows_committed)])
    preempted = set()
    retired = []
    for step in range(800):
        a = rnd.random()
        try:
            if a < 0.12 and len(seqs) < 8:
                s = m.alloc_sequence()
                seqs[s] = 0
            elif a < 0.40 and seqs:
                s = rnd.choice(sorted(seqs))
                if s in open_res or s in preempted:
                    continue
                n = rnd.randrange(1, 12)
                if seqs[s] + n > 190:
                    continue
                r = m.reserve(s, n)
                m.bind_reservation_execution(r.res_id, step)
                open_res[s] = (r.res_id, n)
            elif a < 0.62 and open_res:
                # two-phase commit of a few reservations with ragged prefixes
                picks = rnd.sample(sorted(open_res), k=min(len(open_res), rnd.randrange(1, 3)))
                commits = [(open_res[s][0], rnd.randrange(0, open_res[s][1] + 1)) for s in picks]
                cid = m.prepare_commit(commits)
                if rnd.random() < 0.2:
                    m.abort_prepared_commit(cid)
                    retired.append(m.abort_reservations([c[0] for c in commits]))
                else:
                    retired.append(m.publish_commit(cid))
                    for s, (rid, rows) in zip(picks, commits):
                        seqs[s] += rows
                for s in picks:
                    del open_res[s]
            elif a < 0.68 and open_res:
                s = rnd.choice(sorted(open_res))
                retired.append(m.abort_reservations([open_res.pop(s)[0]]))
            elif a < 0.74 and seqs:
                s = rnd.choice(sorted(seqs))
                if s in open_res or s in preempted:
                    continue
                c = m.publish_fork_sequence_exact(s) if rnd.random() < 0.5 or seqs[s] < 8 else None
                if c is None:
                    t = rnd.randrange(1, seqs[s] // 8 + 1) * 8
                    c = m.publish_fork_sequence_prefix(s, t)
                    seqs[c] = t
                else:
                    seqs[c] = seqs[s]
            elif a < 0.80 and seqs:
                s = rnd.choice(sorted(seqs))
                if s in open_res or s in preempted:
                    continue
                t = rnd.randrange(0, seqs[s] + 1)
                retired.append(m.truncate_sequence(s, t))
                seqs[s] = t
            elif a < 0.85 and seqs:
                s = rnd.choice(sorted(seqs))
                if s in open_res or s in preempted or seqs[s] == 0:
                    continue
                m.preempt_sequence(s)
                retired.append(m.release_preempted_pages(s))
                preempted.add(s)
            elif a < 0.90 and preempted:
                s = rnd.choice(sorted(preempted))
                m.restore_sequence(s)
                preempted.discard(s)
            elif a < 0.96 and seqs:
                s = rnd.choice(sorted(seqs))
                if s in open_res:
                    del open_res[s]
                retired.append(m.free_sequence_pages(s))
                del seqs[s]
                preempted.discard(s)
        except OutOfPages:
            pass
        # confirm retirements at random
        if retired and rnd.random() < 0.5:
            ret = retired.pop(0)
            if ret:
                m.confirm_page_retirement(list(ret.pages))
        m.check_invariants()
        for s, n in seqs.items():
            if s not in preempted:
                assert m.sequence(s).committed_tokens == n, (seed, step, s, m.sequence(s).committed_tokens, n)
    for s in list(seqs):
        retired.append(m.free_sequence_pages(s))
    for ret in retired:
        if ret:
            m.confirm_page_retirement(list(ret.pages))
    m.check_invariants()
    st = m.stats()
    assert st.used_pages == 0 and st.quarantined_pages == 0 and m.free_pages == 24, st



@pytest.mark.parametrize("seed", range(10))
def test_page_manager_soak(seed):
    """Random interleavings of reservations, ragged two-phase commits, aborts, exact and prefix forks, truncation,
    preemption / restore and frees on a 24-page pool: the invariants hold after every operation, every sequence's
    committed length is what the model of the test says, and in the end every page is free."""
    _soak(seed)
