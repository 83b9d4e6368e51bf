"""Failure detection without touching a GPU: heartbeat stragglers, a rank that dies before a collective,
the fp16 overflow watchdog, and the device error word surfacing as an exception (pre-set on the host)."""
import pytest
import torch
import torch.distributed as dist

from common import run_distributed


def test_heartbeat_names_silent_and_stuck_ranks():
    from gpt_neox_b200.obs.heartbeat import Heartbeat
    store = dist.HashStore()
    now = [1000.0]
    clock = lambda: now[0]
    hbs = [Heartbeat(store, r, 4, interval_s=10, clock=clock) for r in range(4)]
    for r in (0, 1, 2):
        hbs[r].beat(5, "forward")
        hbs[r].publish_once()
    bad = hbs[0].stragglers()
    assert [b["rank"] for b in bad] == [3] and bad[0]["reason"] == "no heartbeat"
    hbs[3].beat(5, "forward")
    hbs[3].publish_once()
    assert hbs[0].stragglers() == []
    # rank 2's process dies (publisher silent); rank 1 keeps publishing but its loop is stuck in iteration 5
    now[0] += 40
    for r in (0, 3):
        hbs[r].beat(9, "backward")
        hbs[r].publish_once()
    hbs[1].publish_once()
    bad = {b["rank"]: b["reason"] for b in hbs[0].stragglers()}
    assert set(bad) == {1, 2}
    assert "silent" in bad[2] and "stuck at iteration 5" in bad[1]


def test_heartbeat_thread_publishes():
    import time
    from gpt_neox_b200.obs.heartbeat import Heartbeat
    store = dist.HashStore()
    hb = Heartbeat(store, 0, 1, interval_s=0.05).start()
    hb.beat(3, "optimizer")
    time.sleep(0.3)
    hb.stop()
    assert hb.read_all()[0]["iteration"] == 3


def _rank_dies(rank, world):
    import datetime
    import os
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    t = torch.ones(4)
    dist.all_reduce(t)                       # everyone alive
    if rank == 1:
        os._exit(0)                          # leaves between steps, nothing in flight
    try:
        dist.all_reduce(t)
    except Exception as e:  # noqa: BLE001
        return f"detected: {type(e).__name__}"
    return "not detected"


def test_surviving_rank_gets_an_error_when_a_peer_leaves():
    import torch.multiprocessing as mp
    from common import _worker, free_port
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, _rank_dies, (), ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    assert not any(p.is_alive() for p in procs)
    assert ret[0][0] == "ok" and ret[0][1].startswith("detected"), ret.get(0)


def test_overflow_monitor_raises_after_n_consecutive_skips():
    from gpt_neox_b200.utils.common import OverflowMonitor

    class Opt:
        overflow = True
    mon = OverflowMonitor(Opt(), n=3)
    mon.check(True)
    mon.check(True)
    with pytest.raises(Exception, match="Skipped 3 iterations"):
        mon.check(True)
    mon = OverflowMonitor(Opt(), n=3)
    for s in (True, False, True):
        mon.check(s)                         # not consecutive: no error


@pytest.mark.gpu
def test_device_error_word_becomes_an_exception():
    """A bounded wait that ran out sets the device error word; the host turns it into an exception.  The word
    is pre-set from the host here: no kernel is made to wait."""
    from gpt_neox_b200.ops import _lib
    torch.zeros(1, device="cuda")
    L = _lib.lib()
    assert _lib.read_device_error() == 0
    L.nx_poison_device_error(0x10007)
    with pytest.raises(_lib.DeviceWaitTimeout):
        _lib.raise_on_device_error()
    assert _lib.read_device_error() == 0      # cleared by the read so the context stays usable
    y = torch.ones(8, device="cuda").sum().item()
    assert y == 8


@pytest.mark.gpu
def test_bounded_waits_run_out_return_and_leave_the_context_usable():
    """With a ~1 ms budget, a flag wait on a counter nobody increments and an mbarrier wait nobody arrives on
    both give up: the kernels return, the error word names the code and the site, and after it is cleared an
    ordinary GEMM gives the right answer.  Nothing stalls: each wait ends by itself after its budget."""
    import ctypes as C
    from gpt_neox_b200.ops import _lib
    from gpt_neox_b200.ops.gemm import linear
    L = _lib.lib()
    torch.zeros(1, device="cuda")
    assert _lib.read_device_error() == 0
    _lib.set_wait_budget_cycles(2_000_000)                    # about 1 ms at the clocks seen under load
    try:
        counter = torch.zeros(4, dtype=torch.int32, device="cuda")
        _lib.check(L.nx_wait_counter(_lib.ptr(counter), C.c_uint(5), _lib.stream()), "nx_wait_counter")
        torch.cuda.synchronize()
        v = _lib.read_device_error(clear=True)
        assert (v & 0xff, v >> 8) == (3, 20), hex(v)          # ERR_PEER_TIMEOUT at the delivery-counter wait
        out = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        _lib.check(L.nx_mbar_timeout_probe(_lib.ptr(out), _lib.stream()), "nx_mbar_timeout_probe")
        torch.cuda.synchronize()
        v = _lib.read_device_error(clear=True)
        assert (v & 0xff, v >> 8) == (1, 21), hex(v)          # ERR_WAIT_TIMEOUT at the probe's mbarrier
        assert int(out.item()) == 0                           # the wait reported failure to its caller
        # a counter that is already there does not time out
        counter.fill_(5)
        _lib.check(L.nx_wait_counter(_lib.ptr(counter), C.c_uint(5), _lib.stream()), "nx_wait_counter")
        torch.cuda.synchronize()
        assert _lib.read_device_error() == 0
    finally:
        _lib.set_wait_budget_cycles(0)
    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(384, 256, device="cuda").to(torch.bfloat16)
    y = linear(x, w)
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
    assert _lib.read_device_error() == 0


@pytest.mark.gpu
def test_range_checking_build_records_an_out_of_range_access_and_skips_it():
    """The NEOX_DEBUG_BOUNDS build of the communication kernels: an all-gather whose shard would end beyond the
    registered size of the workspace records {ERR_BOUNDS, site 113} and touches nothing (one rank, its own buffer:
    nothing is out of range in reality, only the registered size is made too small)."""
    import ctypes as C
    import os
    import subprocess
    import sys
    code = r'''
import ctypes as C, torch
from gpt_neox_b200.ops import _lib
L = _lib.lib()
assert L.nx_comm_debug_bounds() == 1
flag = L.nx_comm_flag_bytes()
buf = torch.zeros(flag + 65536, dtype=torch.uint8, device="cuda")
x = torch.full((4096,), 7, dtype=torch.uint8, device="cuda")
ptrs = (C.c_ulonglong * 8)(buf.data_ptr(), *([0] * 7))
L.nx_comm_allgather.argtypes = [C.POINTER(C.c_ulonglong), C.c_ulonglong, C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                                C.c_void_p, C.c_uint, C.c_void_p]
_lib.register_workspace(buf.data_ptr(), flag + 65536)
_lib.check(L.nx_comm_allgather(ptrs, 0, 0, 1, flag, 4096, _lib.ptr(x), 1, _lib.stream()))
torch.cuda.synchronize()
assert _lib.read_device_error() == 0 and int(buf[flag:flag + 4096].sum()) == 7 * 4096
_lib.register_workspace(buf.data_ptr(), flag + 2048)          # pretend the workspace ends in the middle of the shard
buf.zero_()
_lib.check(L.nx_comm_allgather(ptrs, 0, 0, 1, flag, 4096, _lib.ptr(x), 3, _lib.stream()))
torch.cuda.synchronize()
v = _lib.read_device_error()
assert (v & 0xff, v >> 8) == (2, 113), hex(v)
assert int(buf[flag:flag + 2048].sum()) == 7 * 2048 and int(buf[flag + 2048:].sum()) == 0
print("RANGE_CHECK_OK")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    dbg = os.path.join(root, "gpt_neox_b200", "lib", "libneox_b200_dbg.so")
    if not os.path.exists(dbg):
        from gpt_neox_b200.build import build_cuda
        build_cuda(debug_bounds=True)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=root,
                       env=dict(os.environ, NEOX_KERNEL_LIB="debug", PYTHONPATH=root))
    assert "RANGE_CHECK_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
