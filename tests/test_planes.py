"""first_difference of hipinfer_b200/parts/planes.py: run order first, then the order within a layer; shapes; None."""
import torch

from hipinfer_b200.parts import planes


def test_first_difference_walks_in_run_order():
    want = {(-1, "embedding"): torch.ones(2, 4)}
    for l in range(3):
        for n in planes.PLANES:
            want[(l, n)] = torch.full((2, 4), float(l + 1))
    got = {k: v.clone() for k, v in want.items()}
    assert planes.first_difference(got, want, 1e-6) is None
    got[(2, "q")][0, 0] += 1.0
    got[(1, "after_feed_forward")][1, 3] += 0.5
    got[(1, "activation")][1, 3] += 0.25
    key, rel = planes.first_difference(got, want, 1e-6)
    assert key == (1, "activation") and abs(rel - 0.125) < 1e-6
    assert planes.first_difference(got, want, 0.2)[0] == (1, "after_feed_forward")
    got[(0, "mixer_norm")] = torch.ones(3, 4)
    assert planes.first_difference(got, want, 1e-6) == ((0, "mixer_norm"), float("inf"))
    got[(0, "mixer_norm")] = torch.full((2, 4), float("nan"))
    assert planes.first_difference(got, want, 1e-6)[0] == (0, "mixer_norm")


def test_record_is_a_no_op_without_a_dump():
    class B:
        dump = None
        dump_step = 0

    b = B()
    planes.record(b, "q", torch.ones(1))
    planes.record(None, "q", torch.ones(1))
    assert not planes.dumping(b) and not planes.dumping(None)
    b.dump = {}
    x = torch.ones(2)
    planes.record(b, "q", x)
    x += 1
    assert torch.equal(b.dump[(0, "q")], torch.ones(2))
