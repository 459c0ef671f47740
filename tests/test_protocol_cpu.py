"""Host-side checker of the cross-GPU signalling protocol used by the fused collectives.

The device code (ops/csrc/symm.cu) synchronises ranks with epoch flags: rank r writes
``pad[p][slot + r] = epoch`` into every peer p's signal pad and waits until its own pad shows
``>= epoch`` from every peer; every kernel uses two epochs (start = 2k-1, end = 2k). This test
restates that state machine with threads and checks the properties the kernels rely on:
no rank reads a bucket before all ranks published it, no rank overwrites a bucket before all ranks
finished reading it, and a rank that never arrives makes the others time out instead of hang."""
import threading
import time

import pytest


class Pads:
    def __init__(self, W):
        self.W = W
        self.flag = [[0] * W for _ in range(W)]     # flag[owner][source]

    def barrier(self, rank, epoch, timeout_s):
        for p in range(self.W):
            self.flag[p][rank] = epoch               # st.release.sys into peer p's pad
        deadline = time.time() + timeout_s
        for p in range(self.W):
            while self.flag[rank][p] - epoch < 0:    # ld.acquire.sys on the own pad
                if time.time() > deadline:
                    return False
                time.sleep(0)
        return True


def run(W, steps, absent=None, timeout_s=2.0):
    pads = Pads(W)
    bucket = [[0] * W for _ in range(W)]             # bucket[rank][slice] = version written
    log, errors, status = [], [], [0] * W

    def worker(r):
        if r == absent:
            return
        for k in range(1, steps + 1):
            for s in range(W):
                bucket[r][s] = k                     # backward writes this rank's bucket
            if not pads.barrier(r, 2 * k - 1, timeout_s):
                status[r] = 2
                return
            got = [bucket[p][r] for p in range(W)]   # pull own slice from every peer
            if any(g != k for g in got):
                errors.append((r, k, got))
            if not pads.barrier(r, 2 * k, timeout_s):
                status[r] = 2
                return
            log.append((r, k))

    ts = [threading.Thread(target=worker, args=(r,)) for r in range(W)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    return errors, status, log


@pytest.mark.parametrize("W", [2, 4, 8])
def test_epoch_barriers_order_reads_after_writes_and_writes_after_reads(W):
    errors, status, log = run(W, steps=50)
    assert not errors and status == [0] * W and len(log) == W * 50


def test_missing_rank_times_out_with_an_error_status():
    t0 = time.time()
    errors, status, log = run(4, steps=3, absent=2, timeout_s=0.3)
    assert time.time() - t0 < 10
    assert status[2] == 0 and all(status[r] == 2 for r in (0, 1, 3)) and not log
