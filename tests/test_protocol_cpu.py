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


def test_two_streams_need_two_channels():
    """Why every stream that issues barrier kernels has a channel of its own. Rank 0 runs barrier A (epoch 1,
    the optimizer's stream) and barrier B (epoch 2, the compute stream) at the same time; when their signal
    stores land in the order B, A the shared flag word ends at 1 and rank 1's barrier B can never pass, while
    rank 1's barrier A passed before rank 0 had reached it. With one flag word per channel both are exact."""
    # one shared flag word (what rank 1 sees from rank 0): B's store, then A's store
    shared = 0
    shared = 2                       # rank 0, barrier B: st.release epoch 2
    passed_a_early = shared - 1 >= 0        # rank 1 waits in A for epoch 1 and sees 2: passes although A has not run
    shared = 1                       # rank 0, barrier A: st.release epoch 1 overwrites the 2
    b_can_pass = shared - 2 >= 0
    assert passed_a_early and not b_can_pass
    # a flag word per channel, each with its own epoch count
    chan = {1: 0, 3: 0}
    chan[3] = 1                      # barrier B is the first barrier of channel 3
    a_passes_before_a = chan[1] - 1 >= 0
    chan[1] = 1                      # barrier A is the first barrier of channel 1
    assert not a_passes_before_a and chan[1] - 1 >= 0 and chan[3] - 1 >= 0


def test_fused_collectives_count_epochs_per_channel():
    """``FusedCollectives.barrier`` keeps one epoch count per channel (the kernels compare a channel's flag
    words with that channel's count); checked on the bookkeeping alone, with the launch stubbed out."""
    from create_llm_by_cupy_b200.parallel import symm as S

    calls = []

    class Lib:
        def b200_symm_barrier(self, table, W, rank, vr, channel, epoch, wait, stream):
            calls.append((channel, epoch.value))
            return 0

    fc = S.FusedCollectives.__new__(S.FusedCollectives)
    fc.lib, fc.world_size, fc.rank, fc.wait_ns, fc.launches, fc.barrier_epochs = Lib(), 2, 0, 1, 0, {}
    fc._heap = type("H", (), {"table": None})()

    class St:
        cuda_stream = 0

    real_bump, real_check = S.native.bump, S.native.check
    S.native.bump = lambda *a, **k: None
    S.native.check = lambda rc, what: None
    try:
        for ch in (1, 1, 3, 1, 3, 2):
            fc.barrier(St(), channel=ch)
    finally:
        S.native.bump, S.native.check = real_bump, real_check
    assert calls == [(1, 1), (1, 2), (3, 1), (1, 3), (3, 2), (2, 1)]
