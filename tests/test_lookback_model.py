"""CPU model of the chunk-descriptor protocol of the single-pass ("chained") kernels, run under
randomised interleavings.

Every chunk of a chain is a coroutine that performs the kernels' memory operations one at a time
(each ``yield`` is a point where any other chunk may run): wait until its descriptor slot may be
reused, publish its aggregate, look back over its predecessors - window loads first, validity checks
later, exactly the order that lets a slot change hands in between - publish its inclusive state.
The model checks what the kernels rely on: whatever the interleaving and however small the ring, every
chunk ends with the carry a sequential fold gives, bit for bit; a reader that meets a slot taken over
by a later chunk starts over instead of waiting for a tag that cannot come back.
"""
import random

import numpy as np
import pytest

WIN = 4


class Ring:
    """slots x {agg, inc} words; a word is (tag, payload) written and read atomically."""

    def __init__(self, slots):
        self.slots = slots
        self.agg = [(0, None)] * slots
        self.inc = [(0, None)] * slots


def _fold(carry, agg):
    a, h = agg
    return np.float32(a) * np.float32(carry) + np.float32(h)


def chunk_task(k, ring, aggs, h0, out, stats):
    slots = ring.slots
    if k == 0:
        carry = np.float32(h0)
    else:
        # slot reuse rule: the previous owner's successor must have published its inclusive state
        j = k - slots + 1
        while j >= 0 and ring.inc[j % slots][0] != j + 1:
            yield
        ring.agg[k % slots] = (k + 1, aggs[k])
        yield
        restarts = 0
        while True:
            restart = False
            js, carry, top = -1, None, k - 1
            window = {}
            while js < 0 and not restart:
                # all loads of a window first ...
                loaded = {}
                for q in range(WIN):
                    j = top - q
                    if j >= 0:
                        loaded[j] = (ring.inc[j % slots], ring.agg[j % slots])
                        yield
                # ... then the checks, polling where nothing has been published yet
                for q in range(WIN):
                    j = top - q
                    if j < 0 or js >= 0 or restart:
                        continue
                    inc, agg = loaded[j]
                    while inc[0] != j + 1 and agg[0] != j + 1:
                        if inc[0] > j + 1 or agg[0] > j + 1:
                            restart = True
                            break
                        yield
                        inc, agg = ring.inc[j % slots], ring.agg[j % slots]
                    if restart:
                        break
                    if inc[0] == j + 1:
                        js, carry = j, inc[1]
                    else:
                        window[j] = agg[1]
                top -= WIN
            if not restart:
                # aggregates between js and k: those seen in the last window are still in registers, the
                # nearer ones are loaded again - and checked again, their slots may have changed hands
                for j in range(js + 1, k):
                    if j in window and j > top + WIN - 1 - WIN:  # kept from the window that found js
                        agg = window[j]
                    else:
                        tag, agg = ring.agg[j % slots]
                        yield
                        if tag != j + 1:
                            restart = True
                            break
                    carry = _fold(carry, agg)
            if not restart:
                break
            restarts += 1
            stats["restarts"] += 1
            assert restarts < 1000, "look-back does not terminate"
    out[k] = carry
    ring.inc[k % slots] = (k + 1, _fold(carry, aggs[k]))
    yield


@pytest.mark.parametrize("slots", [2, 4, 8, 32])
@pytest.mark.parametrize("in_flight", [3, 9, 24])
def test_look_back_is_exact_under_any_interleaving(slots, in_flight):
    rng = random.Random(100 * slots + in_flight)
    nrng = np.random.default_rng(slots + in_flight)
    stats = {"restarts": 0}
    for trial in range(30):
        n = 60
        aggs = [(np.float32(nrng.uniform(0.8, 1.0)), np.float32(nrng.normal())) for _ in range(n)]
        h0 = np.float32(nrng.normal())
        want, run = [], h0
        for k in range(n):
            want.append(run)
            run = _fold(run, aggs[k])
        ring, out = Ring(slots), {}
        next_k, live = 0, []
        while next_k < n or live:
            while next_k < n and len(live) < in_flight:   # tickets are claimed in order by running workers
                live.append(chunk_task(next_k, ring, aggs, h0, out, stats))
                next_k += 1
            # a stalled front chunk now and then: the others run far ahead of it
            task = live[0] if (len(live) > 1 and rng.random() < 0.02) else rng.choice(live)
            try:
                next(task)
            except StopIteration:
                live.remove(task)
        for k in range(n):
            assert out[k] == want[k], (trial, k)
    RESTARTS[(slots, in_flight)] = stats["restarts"]


RESTARTS = {}


def test_the_model_did_exercise_reused_slots():
    """Runs after the parametrised cases (same module, defined later): some of the small rings must have made
    readers meet slots that had changed hands, or the cases above prove nothing about that path."""
    if not RESTARTS:
        pytest.skip("parametrised cases did not run in this process")
    assert sum(RESTARTS.values()) > 0, RESTARTS
