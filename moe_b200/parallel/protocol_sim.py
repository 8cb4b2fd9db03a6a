"""Host-side simulator of the flag / epoch protocols the peer-memory kernels use.

The kernels in `csrc/comm/allreduce.cu` and `csrc/moe/ep.cu` synchronise through monotonically growing epoch
words in symmetric memory: a producer stores its data, then releases `flag[dst][chan][src] = epoch`; a
consumer spins (bounded) until every source's word is >= its epoch and only then reads.  This module restates
those protocols as small Python coroutines over shared dictionaries and runs them under randomly chosen
interleavings (every `yield` is a point where another rank may run), checking three properties:

* safety: whatever a rank reads was written for the epoch it is waiting for (no stale or early read);
* no overwrite-before-read: a buffer is not rewritten for epoch e+1 while a peer may still read epoch e;
* liveness: every schedule ends (a wait that could never be satisfied shows up as a deadlock here, where on
  the device it would be a bounded wait that runs out).

It exists so that changes to the protocols can be tried on a CPU in milliseconds before any GPU runs them.
"""
from __future__ import annotations

import random
from typing import Callable, Generator, Iterable


class ProtocolError(AssertionError):
    pass


class World:
    """Symmetric memory of `n` ranks: flag words and tagged data cells."""

    def __init__(self, n: int):
        self.n = n
        self.flags: dict = {}   # (owner, chan, src) -> epoch
        self.data: dict = {}    # (owner, name, index) -> tag
        self.reads: list = []

    def flag(self, owner, chan, src) -> int:
        return self.flags.get((owner, chan, src), 0)

    def post(self, owner, chan, src, epoch) -> None:
        if epoch < self.flag(owner, chan, src):
            raise ProtocolError(f"epoch went backwards on flag {(owner, chan, src)}")
        self.flags[(owner, chan, src)] = epoch

    def write(self, owner, name, index, tag) -> None:
        self.data[(owner, name, index)] = tag

    def read(self, owner, name, index, expect) -> None:
        got = self.data.get((owner, name, index))
        if got != expect:
            raise ProtocolError(f"read {(owner, name, index)}: expected {expect}, found {got}")


def wait_all(w: World, owner: int, chan: int, epoch: int, sources: Iterable[int]) -> Generator:
    for s in sources:
        while w.flag(owner, chan, s) < epoch:
            yield ("wait", owner, chan, s, epoch)


def allreduce_rank(w: World, r: int, epoch: int) -> Generator:
    """One bucket of the two-shot reduce: arrive, reduce own slice from every peer, publish, done."""
    n = w.n
    w.write(r, "grad", "all", ("grad", epoch, r))          # backward of this step produced the bucket
    yield
    for d in range(n):                                      # 1. arrive
        w.post(d, 0, r, epoch)
        yield
    yield from wait_all(w, r, 0, epoch, range(n))
    for s in range(n):                                      # 2. read slice r of every peer
        w.read(s, "grad", "all", ("grad", epoch, s))
        yield
    for d in range(n):                                      #    publish the reduced slice everywhere
        w.write(d, "reduced", r, ("sum", epoch, r))
        yield
    for d in range(n):                                      # 3. done
        w.post(d, 1, r, epoch)
        yield
    yield from wait_all(w, r, 1, epoch, range(n))
    for s in range(n):                                      # kernel complete: every slice is final locally
        w.read(r, "reduced", s, ("sum", epoch, s))


def ep_layer_rank(w: World, r: int, e0: int) -> Generator:
    """Forward of one expert-parallel layer: count exchange (epoch e0), row push (e0+1), expert GEMMs whose
    producer waits for the pushes, result scatter + post (e0+2), combine after the owners' posts."""
    n = w.n
    for d in range(n):                                      # counts into every peer's matrix, then the flag
        w.write(d, "cmat", r, ("cnt", e0, r))
        yield
    for d in range(n):
        w.post(d, 10, r, e0)
        yield
    yield from wait_all(w, r, 10, e0, range(n))
    for s in range(n):
        w.read(r, "cmat", s, ("cnt", e0, s))
    for d in range(n):                                      # dispatch: rows into the owners' receive buffers
        w.write(d, "xrecv", r, ("rows", e0 + 1, r))
        yield
    for d in range(n):
        w.post(d, 11, r, e0 + 1)
        yield
    yield from wait_all(w, r, 11, e0 + 1, range(n))         # GEMM producer
    for s in range(n):
        w.read(r, "xrecv", s, ("rows", e0 + 1, s))
        yield
    for d in range(n):                                      # scatter epilogue: results to the token owners
        w.write(d, "yret", r, ("out", e0 + 2, r))
        yield
    for d in range(n):
        w.post(d, 12, r, e0 + 2)
        yield
    yield from wait_all(w, r, 12, e0 + 2, range(n))         # combine
    for s in range(n):
        w.read(r, "yret", s, ("out", e0 + 2, s))


def run(n: int, program: Callable[[World, int], Generator], seed: int = 0, max_steps: int = 1_000_000) -> World:
    """Run one coroutine per rank under a seeded random schedule; raises on a protocol violation or when no
    rank can make progress."""
    rng = random.Random(seed)
    w = World(n)
    procs = {r: program(w, r) for r in range(n)}
    stalled = 0
    for _ in range(max_steps):
        if not procs:
            return w
        r = rng.choice(list(procs))
        try:
            ev = next(procs[r])
        except StopIteration:
            del procs[r]
            stalled = 0
            continue
        if isinstance(ev, tuple) and ev and ev[0] == "wait":
            stalled += 1
            if stalled > 50 * n * n + 1000:  # everybody has been offered the processor many times
                raise ProtocolError(f"deadlock: ranks {sorted(procs)} wait forever, last {ev}")
        else:
            stalled = 0
    raise ProtocolError("schedule did not finish")


def steps_program(kind: str, steps: int, epochs_per_step: int):
    """`steps` consecutive launches with the epoch base advancing like the device counters do."""
    def prog(w: World, r: int):
        base = 1
        for _ in range(steps):
            if kind == "allreduce":
                yield from allreduce_rank(w, r, base)
            else:
                yield from ep_layer_rank(w, r, base)
            base += epochs_per_step
    return prog
