"""The flag / epoch protocols under random interleavings, and the simulator's own ability to catch faults."""
import pytest

from moe_b200.parallel import protocol_sim as P


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("kind,eps", [("allreduce", 1), ("ep", 3)])
def test_protocols_hold_under_random_schedules(n, kind, eps):
    for seed in range(25):
        P.run(n, P.steps_program(kind, steps=3, epochs_per_step=eps), seed=seed)


def test_reusing_an_epoch_is_caught():
    # the second launch does not advance the epoch: a fast rank passes its waits on the first launch's words
    # and reads a slice its peer has not rewritten yet
    def prog(w, r):
        yield from P.allreduce_rank(w, r, 1)
        w.write(r, "grad", "all", None)  # the buffer is being rewritten by the next backward
        yield
        yield from P.allreduce_rank(w, r, 1)

    with pytest.raises(P.ProtocolError):
        for seed in range(200):
            P.run(4, prog, seed=seed)


def test_missing_rank_is_a_deadlock_not_a_pass():
    def prog(w, r):
        if r == 1:
            return
            yield
        yield from P.allreduce_rank(w, r, 1)

    with pytest.raises(P.ProtocolError, match="deadlock"):
        P.run(2, prog, seed=0)


def test_reading_before_the_flag_is_caught():
    def prog(w, r):  # consumer that skips the wait
        w.write(r, "grad", "all", ("grad", 1, r))
        yield
        for s in range(w.n):
            w.read(s, "grad", "all", ("grad", 1, s))
            yield

    with pytest.raises(P.ProtocolError):
        for seed in range(50):
            P.run(4, prog, seed=seed)
