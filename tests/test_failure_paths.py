"""Failure detection without faulting a GPU: a device-side wait that runs out reports a
status code and returns; the host then refuses further collectives on the groups involved;
a rank that raises between steps takes every rank down and training restarts from the last
checkpoint."""
import ctypes
import os

import pytest
import torch

from lbann_b200.ops import native


def test_group_refuses_collectives_after_a_rendezvous_timeout():
    """Host side of the story (no GPU): status 5 poisons every live group of the process."""
    from lbann_b200.parallel import symm
    g = symm.SymmetricGroup(torch.device("cpu"))
    g.barrier_device()                       # single rank: fine
    symm._poison_groups(3)                   # an unrelated status code changes nothing
    g.barrier_device()
    symm._poison_groups(5)
    assert g.poisoned
    with pytest.raises(native.NativeError):
        g.barrier_device()
    with pytest.raises(native.NativeError):
        g.allreduce_small_(torch.zeros(4))


@pytest.mark.gpu
def test_rendezvous_wait_runs_out_and_reports_status():
    """One GPU, one kernel: a group barrier of a pretended two-rank group whose second rank
    does not exist.  Nothing ever sets the flag it waits for; with a 2 ms budget the kernel
    gives up, records "timeout waiting for a flag from another rank" and returns.  The
    context stays usable: the next launches work and report a clean status."""
    lib = native.cuda_lib()
    vpp = ctypes.POINTER(ctypes.c_void_p)
    lib.lb_group_barrier.restype = ctypes.c_int
    lib.lb_group_barrier.argtypes = [vpp, vpp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_void_p]
    lib.lb_comm_pad_bytes.restype = ctypes.c_int
    words = lib.lb_comm_pad_bytes() // 4
    dev = torch.device("cuda")
    pads = [torch.zeros(words, dtype=torch.int32, device=dev) for _ in range(2)]
    ctr = torch.zeros(words, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_void_p * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    assert native.consume_status(False) == 0
    native.set_wait_budget_ns(2_000_000)
    try:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.lb_group_barrier(ptrs, ptrs, 0, 2, 3, ctr.data_ptr(), native.stream_ptr())
        e1.record()
        assert rc == 0
        torch.cuda.synchronize()
        assert 1.0 <= e0.elapsed_time(e1) < 500.0          # gave up after about the budget
        assert native.consume_status(False) == 5
        # rank 0 did announce itself in the "peer's" pad before it started waiting
        assert int(pads[1].sum()) >= 1
    finally:
        native.set_wait_budget_ns(0)
    # the device is fine: an ordinary kernel of the library runs and leaves a clean status
    from lbann_b200.ops.gemm import gemm
    a = torch.randn(128, 64, device=dev).to(torch.bfloat16)
    b = torch.randn(96, 64, device=dev).to(torch.bfloat16)
    y = gemm(a, b, trans_b=True, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.allclose(y, a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)
    assert native.consume_status(False) == 0
    # groups created before the time-out are poisoned by the status listener; reset for later tests
    from lbann_b200.parallel import symm
    for g in list(symm._live_groups):
        g.poisoned = False


def test_rank_failure_aborts_the_job_and_restart_resumes(tmp_path):
    """Two CPU ranks (gloo).  Rank 1 raises between two steps of the second epoch: its
    process ends with a non-zero code, the launcher ends the other rank, the job fails.
    Started again on the same checkpoint directory the job resumes after the first epoch
    and ends with the weights of a run that never failed."""
    import subprocess
    import sys
    from test_distconv_cpu import WORKER, _run
    ref = _run(2, ["abort_restart", str(tmp_path / "ref"), "-1", "3"], str(tmp_path / "ref.json"), timeout=600)
    ck = str(tmp_path / "ck")
    env = dict(os.environ, LBANN_TEST_DEVICE="cpu")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), WORKER,
           "abort_restart", str(tmp_path / "fail.json"), ck, "6", "3"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode != 0                                  # every rank went down
    assert "injected failure on rank 1" in r.stderr
    assert not os.path.exists(tmp_path / "fail.json")
    assert os.path.isdir(ck) and os.listdir(ck)               # the first epoch's checkpoint is there
    got = _run(2, ["abort_restart", ck, "-1", "3"], str(tmp_path / "again.json"), timeout=600)
    assert (got["epoch"], got["step"]) == (ref["epoch"], ref["step"])
    for k, v in ref["weights"].items():
        assert abs(got["weights"][k] - v) <= 1e-6 * max(1.0, abs(v)), k
