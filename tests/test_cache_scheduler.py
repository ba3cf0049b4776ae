"""The cache manager (no page lost, held twice or freed twice, under random orders of requests)
and the scheduler's decisions (admission, portions under the token budget, decoding first,
finishing, and what happens when pages run out). No GPU."""
import random

import pytest

from hipinfer_b200.cache import (CacheError, CacheGroupSpec, CacheManager, OutOfPages, OutOfStateSlots)
from hipinfer_b200.engine.scheduler import AdmissionError, Request, Scheduler
from hipinfer_b200.sampling import SamplingParams

FULL = CacheGroupSpec("full", "full", n_layers=2, kv_heads=2, head_dim=16)
WIN = CacheGroupSpec("win", "window", n_layers=1, kv_heads=1, head_dim=32, window=40)


def test_pages_and_block_tables():
    cm = CacheManager([FULL], page_size=16, num_pages=8, num_state_slots=2)
    cm.add_request("a")
    (slots,) = cm.append("a", 20)
    assert cm.block_table("a", 0) == [0, 1] and slots == list(range(20))
    cm.add_request("b")
    (slots_b,) = cm.append("b", 3)
    assert cm.block_table("b", 0) == [2] and slots_b == [32, 33, 34]
    (more,) = cm.append("a", 13)     # 20 -> 33 tokens: one more page
    assert cm.block_table("a", 0) == [0, 1, 3] and more[:12] == list(range(20, 32)) and more[12] == 48
    assert cm.get("a").length == 33 and cm.free_pages() == [4]
    cm.check()
    cm.free_request("a")
    assert cm.free_pages() == [7]
    cm.add_request("c")
    cm.append("c", 1)
    assert cm.block_table("c", 0) == [0]            # a freed page is used again, lowest id first
    cm.check()


def test_slot_maps_as_arrays_are_the_same_maps():
    """A long portion's slot maps kept as integer arrays (what the runner asks for) hold the same
    slots as the lists, also when the portion starts inside a page and pages are not consecutive."""
    import numpy as np

    def run(as_arrays):
        cm = CacheManager([FULL], page_size=16, num_pages=40, num_state_slots=3)
        out = []
        for rid in ("a", "b"):
            cm.add_request(rid)
        for rid, n in (("a", 5), ("b", 21), ("a", 150), ("b", 3), ("a", 40)):
            (m,) = cm.append(rid, n, as_arrays=as_arrays)
            out.append(np.asarray(m, dtype=np.int64))
        cm.check()
        return out

    for got, want in zip(run(True), run(False)):
        assert got.dtype == np.int64 and got.tolist() == want.tolist()


def test_out_of_pages_changes_nothing_and_misuse_raises():
    cm = CacheManager([FULL], 16, 2, 2)
    cm.add_request("a")
    cm.append("a", 30)
    with pytest.raises(OutOfPages):
        cm.append("a", 5)
    assert cm.get("a").length == 30 and cm.free_pages() == [0]
    assert cm.can_append("a", 2) and not cm.can_append("a", 3)
    with pytest.raises(CacheError):
        cm.add_request("a")
    with pytest.raises(CacheError):
        cm.free_request("zzz")
    cm.add_request("b")
    with pytest.raises(OutOfStateSlots):
        cm.add_request("c")
    cm.free_request("a")
    with pytest.raises(CacheError):
        cm.free_request("a")
    with pytest.raises(CacheError):
        cm.pools[0].release(0)      # freed twice
    cm.check()


def test_state_slots_are_reused_lowest_first():
    cm = CacheManager([FULL], 16, 4, 3)
    s = [cm.add_request(i).state_slot for i in range(3)]
    assert s == [0, 1, 2]
    cm.free_request(1)
    assert cm.add_request("x").state_slot == 1
    cm.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    cm = CacheManager([FULL, WIN], page_size=16, num_pages=[16, 6], num_state_slots=1)
    cm.add_request("a")
    total = 0
    for n in (30, 1, 1, 20, 1, 40, 1, 1, 1):
        cm.append("a", n)
        total += n
        cm.release_behind_window("a")
        table = cm.block_table("a", 1)
        first_needed = max(0, total - 40 + 1)           # the next query is at position `total`
        for lp, page in enumerate(table):
            assert (page == -1) == ((lp + 1) * 16 <= first_needed), (total, lp, table)
        assert all(p >= 0 for p in cm.block_table("a", 0))
        cm.check()
    assert total == 96 and cm.free_pages()[1] >= 2     # 96 tokens fill 6 pages; the window keeps 3 or 4 of them
    cm.free_request("a")
    assert cm.free_pages() == [16, 6]


def test_a_retention_rule_and_planes_registered_from_outside():
    """A kind of group that the package does not know: the first `sink` tokens and the last `window` are kept; what a
    layer keeps per token is a latent and two gate vectors, not keys and values."""
    from hipinfer_b200.cache import register_retention

    def sink_window(spec, q):
        sink = dict(spec.extra)["sink"]
        return ((sink, max(sink, q - spec.window + 1)),)

    with pytest.raises(ValueError, match="kind must be one of"):
        CacheGroupSpec("g", "sink_window_for_test", 1, window=24, planes=(("c", 1, 24),))
    register_retention("sink_window_for_test", sink_window)
    g = CacheGroupSpec("g", "sink_window_for_test", 2, window=24, planes=(("c", 1, 24), ("g", 2, 8)), extra=(("sink", 3),))
    assert g.elements_per_token() == 2 * (24 + 16) and FULL.elements_per_token() == 2 * 2 * 2 * 16
    assert FULL.planes == (("k", 2, 16), ("v", 2, 16))
    with pytest.raises(ValueError, match="distinct names"):
        CacheGroupSpec("g", "full", 1, planes=(("c", 1, 24), ("c", 2, 8)))
    cm = CacheManager([g, FULL], page_size=8, num_pages=[8, 20], num_state_slots=1)
    cm.add_request("a")
    total = 0
    for n in (30, 1, 1, 20, 1, 17, 1, 1, 24):      # 96 tokens = 12 pages on a pool of 8: it works only because pages come back
        cm.append("a", n)
        total += n
        cm.release_behind_window("a")
        for lp, page in enumerate(cm.block_table("a", 0)):
            dead = lp * 8 >= 3 and (lp + 1) * 8 <= total - 24 + 1
            assert (page == -1) == dead, (total, lp)
        assert all(p >= 0 for p in cm.block_table("a", 1))
        cm.check()
    assert cm.block_table("a", 0)[0] >= 0 and cm.free_pages()[0] >= 2
    cm.free_request("a")
    assert total == 96 and cm.free_pages() == [8, 20]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    cm = CacheManager([FULL, WIN], page_size=8, num_pages=[24, 12], num_state_slots=4)
    live, next_id = {}, 0
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and len(live) < 4:
            cm.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif r < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13, 30])
            try:
                maps = cm.append(rid, n)
                assert all(len(m) == n for m in maps)
                live[rid] += n
                cm.release_behind_window(rid)
            except OutOfPages:
                assert not cm.can_append(rid, n)
        elif live:
            rid = rng.choice(list(live))
            cm.free_request(rid)
            del live[rid]
        cm.check()
        for rid, n in live.items():
            assert cm.get(rid).length == n
        # slots of different requests never collide
        seen = set()
        for rid in live:
            for p in cm.block_table(rid, 0):
                assert p not in seen
                seen.add(p)
    for rid in list(live):
        cm.free_request(rid)
    assert cm.free_pages() == [24, 12] and cm.slots.free_count == 4


# ------------------------------------------------------------------------------------------
# scheduler
# ------------------------------------------------------------------------------------------
def make(num_pages=64, page_size=16, max_seqs=4, budget=32, max_len=512):
    cm = CacheManager([FULL], page_size, num_pages, max_seqs)
    return cm, Scheduler(cm, max_seqs, budget, max_len, eos_token_ids=(9,))


def req(rid, n_prompt, n_new, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(max_new_tokens=n_new, **kw))


def run_step(cm, sch, token=5):
    """What the engine does around a step, with the cache manager standing in for the device."""
    sched = sch.schedule()
    for s in sched:
        if not cm.has_request(s.request.request_id):
            cm.add_request(s.request.request_id)
        assert cm.get(s.request.request_id).length == s.start
        cm.append(s.request.request_id, s.n)
    cm.check()
    toks = [token for s in sched if s.samples]
    return sched, sch.update(sched, toks)


def test_prompt_is_cut_into_portions_under_the_budget():
    cm, sch = make(budget=32)
    sch.add(req("a", 70, 2))
    s1, _ = run_step(cm, sch)
    assert [(s.start, s.n, s.samples) for s in s1] == [(0, 32, False)]
    s2, _ = run_step(cm, sch)
    assert [(s.start, s.n, s.samples) for s in s2] == [(32, 32, False)]
    s3, done = run_step(cm, sch)
    assert [(s.start, s.n, s.samples) for s in s3] == [(64, 6, True)] and not done
    s4, done = run_step(cm, sch)
    assert [(s.start, s.n, s.samples) for s in s4] == [(70, 1, True)]
    assert [r.request_id for r in done] == ["a"] and done[0].output == [5, 5] and done[0].finish_reason == "length"
    assert cm.free_pages() == [64] and not sch.has_work()


def test_decoding_requests_come_first_and_prompts_share_the_rest():
    cm, sch = make(budget=16)
    sch.add(req("a", 4, 8))
    run_step(cm, sch)                  # a is now decoding
    sch.add(req("b", 40, 4))
    sch.add(req("c", 10, 4))
    s, _ = run_step(cm, sch)
    assert [(x.request.request_id, x.n) for x in s] == [("a", 1), ("b", 15)]
    s, _ = run_step(cm, sch)
    assert [(x.request.request_id, x.n) for x in s] == [("a", 1), ("b", 15)]
    s, _ = run_step(cm, sch)           # b's last 10 prompt tokens, then c gets what is left
    assert [(x.request.request_id, x.start, x.n, x.samples) for x in s] == [("a", 6, 1, True), ("b", 30, 10, True),
                                                                           ("c", 0, 5, False)]


def test_admission_is_first_come_first_served_and_bounded_by_slots():
    cm, sch = make(max_seqs=2, budget=64)
    for i in range(4):
        sch.add(req(i, 5, 3))
    s, _ = run_step(cm, sch)
    assert [x.request.request_id for x in s] == [0, 1]
    while len(sch.finished) < 2:
        s, _ = run_step(cm, sch)
    s, _ = run_step(cm, sch)
    assert sorted(x.request.request_id for x in s) == [2, 3]


def test_requests_that_can_never_fit_are_refused():
    cm, sch = make(num_pages=4, page_size=16, max_len=100)
    with pytest.raises(AdmissionError, match="longest sequence"):
        sch.add(req("long", 90, 20))
    with pytest.raises(AdmissionError, match="pages"):
        sch.add(req("big", 60, 10))      # 69 cached tokens = 5 pages > 4
    with pytest.raises(AdmissionError, match="empty"):
        sch.add(Request("e", [], SamplingParams()))
    sch.add(req("ok", 60, 5))            # 64 cached tokens = 4 pages


def test_stop_tokens_and_eos():
    cm, sch = make()
    sch.add(req("a", 3, 10, stop_token_ids=(5,)))
    sch.add(req("b", 3, 3, ignore_eos=False))
    _, done = run_step(cm, sch, token=5)
    assert [r.request_id for r in done] == ["a"] and done[0].finish_reason == "stop"
    _, done = run_step(cm, sch, token=9)
    assert [r.request_id for r in done] == ["b"] and done[0].finish_reason == "stop"


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    # 6 pages of 16: two requests of 40 prompt tokens (3 pages each) fill the pool exactly at 48 tokens each
    cm, sch = make(num_pages=6, page_size=16, budget=128, max_seqs=2)
    sch.add(req("old", 40, 30))
    sch.add(req("young", 40, 30))
    run_step(cm, sch)                                # both prefilled: 3 + 3 pages
    assert cm.free_pages() == [0]
    for _ in range(8):                               # 41..48 tokens: still 3 pages each
        s, _ = run_step(cm, sch)
        assert [x.request.request_id for x in s] == ["old", "young"]
    assert sch.n_preemptions == 0
    s, _ = run_step(cm, sch)                         # the 49th token needs a 4th page: none free
    assert [x.request.request_id for x in s] == ["old"]
    young = sch.waiting[0]
    assert young.request_id == "young" and young.n_cached == 0 and young.preemptions == 1
    assert len(young.output) == 9 and not cm.has_request("young")
    assert sch.n_preemptions == 1
    # old runs on alone until it finishes; young cannot come back before there is room for all its tokens
    readmit, steps = None, 0
    while readmit is None and steps < 100:
        s, _ = run_step(cm, sch)
        steps += 1
        readmit = next((x for x in s if x.request.request_id == "young"), None)
        if readmit is None:
            assert [x.request.request_id for x in s] == ["old"]
    assert readmit.start == 0 and readmit.n == 40 + 9 and readmit.samples   # prompt + produced so far, computed again
    while sch.has_work():
        run_step(cm, sch)
    assert {r.request_id: len(r.output) for r in sch.finished} == {"old": 30, "young": 30}
    assert cm.free_pages() == [6] and cm.slots.free_count == 2


def test_a_preempted_request_comes_back_while_others_still_run():
    """A victim waits only until its next portion fits: not until every running request has ended."""
    cm, sch = make(num_pages=12, page_size=16, budget=64, max_seqs=3)
    sch.add(req("a", 60, 40))         # 4 pages, grows to 7
    sch.add(req("b", 60, 5))          # 4 pages, ends early
    sch.add(req("c", 60, 40))         # 4 pages: the pool is full after the three prompts
    for _ in range(3):
        run_step(cm, sch)
    assert cm.free_pages() == [0] and len(sch.running) == 3
    back = None
    for step in range(60):
        s, _ = run_step(cm, sch)
        ids = [x.request.request_id for x in s]
        if sch.n_preemptions and back is None and "c" in ids:
            back = step
            assert "a" in ids, "the victim came back only after the others had ended"
            assert next(x for x in s if x.request.request_id == "c").start == 0
            break
    assert sch.n_preemptions >= 1 and back is not None
    while sch.has_work():
        run_step(cm, sch)
    assert {r.request_id: len(r.output) for r in sch.finished} == {"a": 40, "b": 5, "c": 40}
    assert cm.free_pages() == [12] and cm.slots.free_count == 3


def test_a_request_finished_while_it_waits_is_never_scheduled_again():
    """finish() on a request that a later schedule() preempted (a stop token read back one step late):
    it leaves the waiting queue, is reported once and produces nothing more."""
    cm, sch = make(num_pages=6, page_size=16, budget=128, max_seqs=2)
    sch.add(req("old", 40, 30))
    sch.add(req("young", 40, 30))
    for _ in range(9):
        run_step(cm, sch)
    s, _ = run_step(cm, sch)                         # young is preempted here
    young = sch.waiting[0]
    assert young.request_id == "young" and sch.n_preemptions == 1
    n_out = len(young.output)
    sch.finish(young, "stop")
    assert young not in sch.waiting and young.status == "finished"
    while sch.has_work():
        s, _ = run_step(cm, sch)
        assert all(x.request.request_id == "old" for x in s)
    assert len(young.output) == n_out
    assert [r.request_id for r in sch.finished].count("young") == 1
    assert cm.free_pages() == [6] and cm.slots.free_count == 2


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_nothing_lost(seed):
    rng = random.Random(seed)
    cm, sch = make(num_pages=20, page_size=8, max_seqs=4, budget=24, max_len=200)
    want = {}
    for i in range(12):
        n_prompt, n_new = rng.randint(1, 70), rng.randint(1, 40)
        try:
            sch.add(req(i, n_prompt, n_new))
            want[i] = n_new
        except AdmissionError:
            assert -(-(n_prompt + n_new - 1) // 8) > 20
    steps = 0
    while sch.has_work():
        sched, _ = run_step(cm, sch)
        assert sched, "work left but nothing scheduled"
        assert sum(s.n for s in sched) <= 24 and len(sch.running) <= 4
        steps += 1
        assert steps < 5000
    assert {r.request_id: len(r.output) for r in sch.finished} == want
    assert cm.free_pages() == [20] and cm.slots.free_count == 4
