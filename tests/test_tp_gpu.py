"""Tensor parallelism on real GPUs (needs at least two): two ranks, NCCL, logits against the unsharded oracle."""
import os
import socket

import numpy as np
import pytest

from juno_b200 import synth

pytestmark = pytest.mark.gpu
ARCH = synth.Arch(hidden=512, n_layers=2, n_heads=4, n_kv_heads=2, inter=1024, vocab=1024, rope_theta=500000.0)


def _gpu_count():
    from juno_b200.matvec import GpuContext
    return GpuContext.device_count()


def _worker(rank, world, nccl_id, q, push):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["JUNO_TP_PUSH"] = "1" if push else "0"
    from juno_b200.handler import B200TransformerHandler
    from juno_b200.matvec import GpuContext
    ctx = GpuContext(rank)
    h = B200TransformerHandler(ARCH, ctx, max_batch=2, max_seqs=2, max_ctx=32, kv_dtype="f32", tp_rank=rank,
                               tp_world=world, nccl_id=nccl_id)
    h.load(synth.random_model(ARCH, 21, norm="random"))
    outs = []
    toks = [[5, 900], [17, 3], [512, 77], [1, 2]]
    for p, t in enumerate(toks):
        logits, ids = h.forward_batch(["a", "b"], [[t[0]], [t[1]]], [p, p], want_logits=True, want_argmax=True)
        outs.append((logits.copy(), ids.copy()))
    greedy = h.decode_greedy(["a", "b"], [7, 8], [len(toks), len(toks)], 6)
    h.release_gpu_resources()
    q.put((rank, outs, greedy))


@pytest.mark.parametrize("push", [True, False], ids=["peer-push", "nccl"])
def test_two_gpu_tensor_parallel_matches_oracle(oracle, push):
    """Both exchanges of the row-parallel partial products: stores into peer-mapped inboxes by the producing kernel
    (the default for up to eight sequences), and NCCL all-reduce."""
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from juno_b200.handler import B200TransformerHandler
    from modelutil import build_pair
    nccl_id = B200TransformerHandler.nccl_unique_id()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=_worker, args=(r, 2, nccl_id, q, push)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(2)], key=lambda r: r[0])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    om, _ = build_pair(oracle, ARCH, 21, kv_dtype="f32", max_ctx=32, engine=False)
    sa, sb = om.new_seq(), om.new_seq()
    toks = [[5, 900], [17, 3], [512, 77], [1, 2]]
    for p, t in enumerate(toks):
        ra, rb = om.forward(sa, t[0], p), om.forward(sb, t[1], p)
        for rank in range(2):
            logits, ids = res[rank][1][p]
            assert np.abs(logits[0] - ra).max() <= 1e-3 * np.abs(ra).max()
            assert np.abs(logits[1] - rb).max() <= 1e-3 * np.abs(rb).max()
            assert ids[0] == oracle.greedy(ra) and ids[1] == oracle.greedy(rb)
    assert np.array_equal(res[0][2], res[1][2])  # both ranks pick the same tokens


def _worker_missing_peer(rank, world, nccl_id, q, done, push=True):
    """Rank 1 stops taking part between steps (nothing of it in flight; the process and its buffers stay until the
    test is over); rank 0 runs one more step alone."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["JUNO_TP_PUSH"] = "1" if push else "0"
    os.environ["JUNO_NCCL_TIMEOUT_S"] = "3"
    from juno_b200 import _lib
    from juno_b200.handler import B200TransformerHandler
    from juno_b200.matvec import GpuContext
    ctx = GpuContext(rank)
    h = B200TransformerHandler(ARCH, ctx, max_batch=1, max_seqs=1, max_ctx=32, kv_dtype="f32", tp_rank=rank, tp_world=world,
                               nccl_id=nccl_id)
    h.load(synth.random_model(ARCH, 21))
    first = h.decode_greedy(["a"], [5], [0], 2)  # both ranks: two steps together
    q.put(("ready", rank, first.tolist()))
    if rank == 1:
        done.wait(120)  # takes no further part; rank 0 may still store into this rank's inbox, so the memory stays
        return
    import time
    time.sleep(1.0)
    if push and h.tp_mode() != 2:  # no peer mapping on this system: nothing to test in this mode
        q.put(("result", rank, "skipped: NCCL mode", 0.0))
        return
    t0 = time.time()
    try:
        h.decode_greedy(["a"], [7], [2], 1)
        q.put(("result", rank, "no error", time.time() - t0))
    except _lib.JunoError as e:
        msg, dt = f"rc={e.rc}: {e}", time.time() - t0
        if not push:  # the communicator is gone: the model refuses further steps instead of hanging in them
            try:
                h.decode_greedy(["a"], [7], [2], 1)
                msg += " | second step: no error"
            except _lib.JunoError as e2:
                msg += f" | second step: rc={e2.rc}"
        q.put(("result", rank, msg, dt))


def test_missing_rank_times_out_instead_of_hanging():
    """Failure detection without a GPU fault: a rank that stops taking part between steps makes the other rank's
    bounded waits (for partial products, for the greedy pick) run out; the step returns JUNO_ERR_TIMEOUT within a
    few seconds and the context stays usable.  No collective call is in the greedy step, so nothing can hang."""
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from juno_b200 import _lib
    from juno_b200.handler import B200TransformerHandler
    nccl_id = B200TransformerHandler.nccl_unique_id()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    done = mpc.Event()
    procs = [mpc.Process(target=_worker_missing_peer, args=(r, 2, nccl_id, q, done)) for r in range(2)]
    for p in procs:
        p.start()
    msgs = []
    try:
        for _ in range(3):
            msgs.append(q.get(timeout=90))
    except Exception:
        pass
    finally:
        done.set()
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.kill()
    assert len(msgs) == 3, f"a rank never reported: {msgs}"
    ready = [m for m in msgs if m[0] == "ready"]
    assert len(ready) == 2 and ready[0][2] == ready[1][2]
    res = [m for m in msgs if m[0] == "result"][0]
    if res[2].startswith("skipped"):
        pytest.skip(res[2])
    assert f"rc={_lib.ERR_TIMEOUT}" in res[2] and "did not deliver" in res[2], res
    assert res[3] < 30.0, res


def test_missing_rank_in_nccl_mode_is_ended_by_the_watchdog():
    """The same failure with the NCCL exchange: the all-reduce of the lonely rank can never complete; the step's wait
    polls the stream with a deadline (JUNO_NCCL_TIMEOUT_S=3 here), aborts the communicator and returns
    JUNO_ERR_TIMEOUT; later steps are refused with JUNO_ERR_NCCL.  Nothing faults: the abort ends NCCL's own kernel."""
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from juno_b200 import _lib
    from juno_b200.handler import B200TransformerHandler
    nccl_id = B200TransformerHandler.nccl_unique_id()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    done = mpc.Event()
    procs = [mpc.Process(target=_worker_missing_peer, args=(r, 2, nccl_id, q, done, False)) for r in range(2)]
    for p in procs:
        p.start()
    msgs = []
    try:
        for _ in range(3):
            msgs.append(q.get(timeout=90))
    except Exception:
        pass  # judged below: a missing message means the watchdog did not end the step
    finally:
        done.set()
        for p in procs:
            p.join(30)
            if p.is_alive():
                p.kill()  # this exact child: a wait for the vanished peer must not hold the suite
    res = [m for m in msgs if m[0] == "result"]
    assert res, f"the lonely rank never returned from its step: {msgs}"
    res = res[0]
    assert f"rc={_lib.ERR_TIMEOUT}" in res[2] and "communicator was aborted" in res[2], res
    assert f"second step: rc={_lib.ERR_NCCL}" in res[2], res
    assert res[3] < 30.0, res
