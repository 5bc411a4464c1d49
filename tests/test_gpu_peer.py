"""The peer-store exchange kernels (qx_cuda_peer_push / qx_cuda_peer_wait).

On one GPU the "peers" are separate buffers of the same device: the push kernel's data movement,
its data-before-flag publication and the wait kernel's bounded wait can all be checked without a
second GPU.  No kernel here waits for another launch: a wait either finds its flags already set by
a kernel that completed earlier on the stream, or waits for a flag that nothing sets and must give
up after its limit (status 1), after which later waits on the same status word return at once.
The multi-GPU form (two ranks, symmetric memory) runs when the machine has at least two GPUs."""
import ctypes
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from quixicore_metal_b200 import _lib
    return _lib, _lib.lib()


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_push_copies_the_slot_to_every_peer_and_publishes_the_step():
    _l, L = _lib()
    world, me, n = 3, 1, 4096 + 12                       # floats; a multiple of 4
    src = torch.randn(n, device="cuda")
    peers = [torch.zeros(n, device="cuda") for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(world)]
    tickets = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for step in (1, 2, 7):
        src.normal_()
        r = L.qx_cuda_peer_push(st, src.data_ptr(), 4 * n, _ptrs(peers), _ptrs(flags), world, me, step, tickets.data_ptr())
        assert r.code == 0, r.detail
        torch.cuda.synchronize()
        for q in range(world):
            if q == me:
                assert not peers[q].any() and int(flags[q][me]) == 0      # nothing is written to the own slot
            else:
                assert torch.equal(peers[q], src) and int(flags[q][me]) == step
        assert int(tickets) == 0                                          # reset for the next launch


def test_wait_passes_on_published_flags_and_gives_up_on_a_missing_one():
    _l, L = _lib()
    world, me = 4, 2
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    flags[:world] = torch.tensor([5, 5, 0, 6], dtype=torch.int32)        # own entry is never read; a peer may be ahead
    r = L.qx_cuda_peer_wait(st, flags.data_ptr(), world, me, 5, 1000, status.data_ptr())
    assert r.code == 0, r.detail
    torch.cuda.synchronize()
    assert int(status) == 0
    # rank 1 never publishes step 6: the wait runs out after its limit and reports it
    t0 = time.time()
    r = L.qx_cuda_peer_wait(st, flags.data_ptr(), world, me, 6, 50, status.data_ptr())
    assert r.code == 0
    torch.cuda.synchronize()
    assert int(status) == 1 and time.time() - t0 < 5.0
    # a later wait on the same status word does not wait again
    t0 = time.time()
    L.qx_cuda_peer_wait(st, flags.data_ptr(), world, me, 9, 2000, status.data_ptr())
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert L.qx_cuda_device_error() == 0                                  # the library-wide flag is not involved


def test_push_and_wait_argument_checks():
    _l, L = _lib()
    buf = torch.zeros(64, device="cuda")
    fl = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    p = _ptrs([buf, buf])
    f = _ptrs([fl, fl])
    assert _l.STATUS_NAMES[L.qx_cuda_peer_push(st, buf.data_ptr(), 24, p, f, 2, 0, 1, fl.data_ptr()).code] == "invalid_shape"
    assert _l.STATUS_NAMES[L.qx_cuda_peer_push(st, buf.data_ptr(), 64, p, f, 17, 0, 1, fl.data_ptr()).code] == "invalid_argument"
    assert _l.STATUS_NAMES[L.qx_cuda_peer_wait(st, fl.data_ptr(), 2, 2, 1, 100, fl.data_ptr()).code] == "invalid_argument"
    assert _l.STATUS_NAMES[L.qx_cuda_peer_wait(st, fl.data_ptr(), 2, 0, 1, 0, fl.data_ptr()).code] == "invalid_argument"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_peer_exchange_gives_the_nccl_ids():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "_peer_exchange_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "peer exchange ok" in out.stdout


def test_single_launch_allreduce_with_three_ranks_on_one_gpu():
    """All three ranks' buffers live on this GPU and run as ONE cooperative launch (ranks that wait for
    one another cannot be separate launches on one GPU): every rank returns residual + the partials
    summed in rank order, bit-identical, over consecutive steps (both buffer halves), for sizes of one
    and of several CTAs per rank."""
    _l, L = _lib()
    W = 3
    for n in (2048, 8192 * 5, 6):
        bufs = [torch.zeros(4 * W * n, device="cuda") for _ in range(W)]
        counters = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
        tickets = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
        status = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
        st = torch.cuda.current_stream().cuda_stream
        for step in range(1, 5):
            parts = [torch.randn(n, device="cuda") for _ in range(W)]
            res = [torch.randn(n, device="cuda").bfloat16() for _ in range(W)]
            outs = [torch.empty(n, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
            rc = L.qx_cuda_peer_allreduce_local(st, _ptrs(parts), _ptrs(res), _ptrs(outs), n, _ptrs(bufs), W,
                                                _ptrs(counters), _ptrs(tickets), _ptrs(status), _l.DTYPE_BF16, 1000)
            assert rc.code == 0, rc.detail
            torch.cuda.synchronize()
            total = (parts[0] + parts[1]) + parts[2]
            for r in range(W):
                assert torch.equal(outs[r], (total + res[r].float()).bfloat16()), (n, step, r)
                assert int(counters[r]) == step and int(tickets[r]) == 0 and int(status[r]) == 0


def test_single_launch_allreduce_gives_up_when_the_peers_never_come():
    """Rank 0 of three runs alone: its wait for the words of ranks 1 and 2 (which nothing writes) ends
    at its limit, the status word says so, the context stays usable and a later call does not wait."""
    _l, L = _lib()
    W, n = 3, 4096
    buf = torch.zeros(4 * W * n, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    tickets = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    part = torch.randn(n, device="cuda")
    res = torch.randn(n, device="cuda").bfloat16()
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    rc = L.qx_cuda_peer_allreduce(st, part.data_ptr(), res.data_ptr(), out.data_ptr(), n, _ptrs([buf] * W), W, 0,
                                  counter.data_ptr(), tickets.data_ptr(), status.data_ptr(), _l.DTYPE_BF16, 20)
    assert rc.code == 0, rc.detail
    torch.cuda.synchronize()
    assert int(status) == 1 and int(counter) == 1 and time.time() - t0 < 5.0
    t0 = time.time()
    rc = L.qx_cuda_peer_allreduce(st, part.data_ptr(), res.data_ptr(), out.data_ptr(), n, _ptrs([buf] * W), W, 0,
                                  counter.data_ptr(), tickets.data_ptr(), status.data_ptr(), _l.DTYPE_BF16, 5000)
    torch.cuda.synchronize()
    assert rc.code == 0 and int(counter) == 2 and time.time() - t0 < 1.0
    assert torch.equal(torch.ones(4, device="cuda") * 2, torch.full((4,), 2.0, device="cuda"))   # the context still works


def test_single_launch_gather_with_three_ranks_on_one_gpu():
    """All-gather of small slots by words that carry their step number: three ranks on this GPU as ONE
    cooperative launch; afterwards every rank's gather buffer holds every rank's slot bit for bit
    (NaN payloads and int32 ids travelling as float bits included), over consecutive steps."""
    _l, L = _lib()
    W = 3
    for n in (2, 200, 40000):
        words = [torch.zeros(4 * W * n, device="cuda") for _ in range(W)]
        status = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(W)]
        st = torch.cuda.current_stream().cuda_stream
        for step in range(1, 5):
            slots = [torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), dtype=torch.int32, device="cuda") for _ in range(W)]
            gathers = [torch.zeros(W * n, dtype=torch.int32, device="cuda") for _ in range(W)]
            for r in range(W):
                gathers[r][r * n:(r + 1) * n] = slots[r]
            rc = L.qx_cuda_peer_gather_local(st, _ptrs(gathers), n, _ptrs(words), W, step, 1000, _ptrs(status))
            assert rc.code == 0, rc.detail
            torch.cuda.synchronize()
            want = torch.cat(slots)
            for r in range(W):
                assert torch.equal(gathers[r], want), (n, step, r)
                assert int(status[r]) == 0


def test_single_launch_gather_gives_up_when_the_peers_never_come():
    _l, L = _lib()
    W, n = 3, 512
    words = torch.zeros(4 * W * n, device="cuda")
    gather = torch.zeros(W * n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    rc = L.qx_cuda_peer_gather(st, gather.data_ptr(), n, _ptrs([words] * W), W, 0, 1, 20, status.data_ptr())
    assert rc.code == 0, rc.detail
    torch.cuda.synchronize()
    assert int(status) == 1 and time.time() - t0 < 5.0
    t0 = time.time()
    rc = L.qx_cuda_peer_gather(st, gather.data_ptr(), n, _ptrs([words] * W), W, 0, 2, 5000, status.data_ptr())
    torch.cuda.synchronize()
    assert rc.code == 0 and time.time() - t0 < 1.0
