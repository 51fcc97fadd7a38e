"""GPU tests of the fused compressed all-reduce. Single-GPU cases run in
process; multi-GPU cases launch one worker per GPU with torchrun."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from gcow_b200 import _native
from gcow_b200.codec import ZfpParams
from gcow_b200.comm import CompressedAllReduce, CollectiveTimeout, allreduce_oracle
from gcow_b200.config import GcowConfig

HERE = os.path.dirname(os.path.abspath(__file__))


def gen(seed, n):
    return (np.random.default_rng(seed).standard_normal(n) * 1e-3).astype(np.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("rate", [4, 8, 16, 32])
def test_single_rank_equals_oracle(rate):
    p = ZfpParams.from_rate(rate, 1)
    ar = CompressedAllReduce(1 << 20, GcowConfig(rate=rate, comm_ctas=64))
    for n in (3, 4099, 1 << 20, (1 << 20) + (1 << 19) + 5):   # the last one is split into two launches
        x = gen(n, n)
        pieces = [x[i:i + (1 << 20)] for i in range(0, n, 1 << 20)]
        ref = np.concatenate([allreduce_oracle(q[None], p, "twoshot", 0) for q in pieces])
        y = ar(torch.from_numpy(x).cuda(), variant="twoshot")
        ar.check()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
        # the default on one rank is a single round trip D(E(x)), as the reference applies to the local gradient
        assert ar.pick_variant(n) == "oneshot"
        one = np.concatenate([allreduce_oracle(q[None], p, "oneshot", 0) for q in pieces])
        y1 = ar(torch.from_numpy(x).cuda())
        ar.check()
        assert np.array_equal(y1.cpu().numpy().view(np.uint32), one.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("cap,tol", [(4, 1e-2), (8, 1e-3), (16, 1e-6), (32, 1e-4)])
def test_accuracy_mode_single_rank_equals_oracle(cap, tol):
    """Fixed accuracy with a bit cap (the sparse variant): bit-exact against the host model at the same four codec
    parameters; blocks below the tolerance come back as zeros; error feedback keeps what was dropped."""
    ar = CompressedAllReduce(1 << 20, GcowConfig(mode="accuracy", tolerance=tol, rate=cap, comm_ctas=64))
    assert ar.pick_variant(123) == "sparse" and ar.params.minbits == 1 and ar.params.maxbits == 4 * cap
    for n in (3, 4099, 1 << 20, (1 << 20) + 77):
        x = gen(n + cap, n)
        x[n // 2:] *= np.float32(1e-5)                       # far below every tolerance used here
        pieces = [x[i:i + (1 << 20)] for i in range(0, n, 1 << 20)]
        ref = np.concatenate([allreduce_oracle(q[None], ar.params, "twoshot", 0) for q in pieces])
        y = ar(torch.from_numpy(x).cuda())
        ar.check()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
        if n > 8:
            assert not ref[n // 2 + 4:].any() and ref[: n // 2].any()
    x = torch.from_numpy(gen(5, 4096)).cuda()
    res = torch.zeros_like(x)
    y = ar(x.clone(), residual=res)
    ar.check()
    p1 = ZfpParams(ar.params.minbits, ar.params.maxbits, ar.params.maxprec, ar.params.minexp)
    once = allreduce_oracle(x.cpu().numpy()[None], p1, "oneshot", 0)        # D(E(x)): what this rank's code kept
    assert np.array_equal(res.cpu().numpy(), x.cpu().numpy() - once)
    assert ar.wire_bytes() == 0                                               # one rank: nothing leaves the GPU


@pytest.mark.gpu
def test_rate_2_is_the_header_only_floor():
    """9 bits per block keep no bit plane: D(E(x)) = 0, and so is the reduced result (as in the host model)."""
    p = ZfpParams.from_rate(2, 1)
    assert p.maxbits == 9
    x = gen(3, 4099)
    ref = allreduce_oracle(x[None], p, "twoshot", 0)
    assert not ref.any()
    ar = CompressedAllReduce(1 << 16, GcowConfig(rate=2))
    y = ar(torch.from_numpy(x).cuda())
    ar.check()
    assert not y.cpu().numpy().any()


@pytest.mark.gpu
def test_out_of_place_and_stamps():
    ar = CompressedAllReduce(1 << 18, GcowConfig(rate=8, comm_ctas=16))
    ar.enable_tracing()
    x = torch.from_numpy(gen(1, 1 << 18)).cuda()
    keep = x.clone()
    out = torch.empty_like(x)
    ar(x, out=out)
    ar.check()
    assert torch.equal(x, keep)
    st = ar.phase_stamps()
    assert st.shape == (16, 4) and bool((st[:, 3] >= st[:, 0]).all()) and int(st.min()) > 0


@pytest.mark.gpu
def test_wait_that_nothing_satisfies_returns_a_status():
    """A bounded wait on a flag nobody sets must end by itself with a time-out
    record, and the context must stay usable."""
    lib = _native.cuda()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    assert lib.gcow_ar_wait_probe(flag.data_ptr(), 7, 50_000_000, status.data_ptr(), status[8:].data_ptr(), s) == 0
    torch.cuda.synchronize()
    dt = time.time() - t0
    rec = status.cpu().tolist()
    assert rec[0] == 1 and rec[4] == 7 and rec[5] == 0 and rec[8] == 1   # time-out, expected 7, saw 0, abort raised
    assert 0.03 < dt < 5.0
    # context still fine, and a satisfied wait returns clean
    status.zero_()
    flag.fill_(7)
    assert lib.gcow_ar_wait_probe(flag.data_ptr(), 7, 50_000_000, status.data_ptr(), status[8:].data_ptr(), s) == 0
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def _run_workers(nproc, extra_env=None, script="mp_allreduce_worker.py", timeout=900):
    out = os.path.join(HERE, f"_mp_out_{nproc}.json")
    if os.path.exists(out):
        os.remove(out)
    env = dict(os.environ, GCOW_TEST_OUT=out, MASTER_ADDR="127.0.0.1")
    env.update(extra_env or {})
    port = 29500 + (os.getpid() % 400) + nproc
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    res = None
    if os.path.exists(out):
        with open(out) as f:
            res = json.load(f)
        os.remove(out)
    return proc, res


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_multi_gpu_bit_exact(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    proc, res = _run_workers(nproc)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert res is not None and res["world"] == nproc and not any(res["fails"])


@pytest.mark.multigpu
def test_multi_gpu_ipc_backend():
    proc, res = _run_workers(2, {"GCOW_COMM_BACKEND": "ipc"})
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert res["backend"] == "ipc" and not any(res["fails"])


@pytest.mark.multigpu
def test_multi_gpu_256mb_buffer_matches_host_model():
    """One 256 MB gradient buffer per rank at 4/8/16 bit/value on every visible GPU (2, 4 or 8), bit for bit
    against decode-sum-encode on the host."""
    n = torch.cuda.device_count()
    nproc = 8 if n >= 8 else 4 if n >= 4 else 2
    proc, res = _run_workers(nproc, {"GCOW_TEST_BIG": "1"}, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert res is not None and res["world"] == nproc and not any(res["fails"])


@pytest.mark.multigpu
def test_late_peer_times_out_on_both_ranks_then_recovers():
    """A rank that reaches its launch 300 ms late, with 50 ms waits: both ranks get a time-out record instead of a
    hang, the next call is bit-exact again, and the training hook's safe mode finishes the step with NCCL. Plain peer
    loads and stores (IPC backend, no multicast object bound), NVLS off in NCCL."""
    proc, res = _run_workers(2, {"GCOW_COMM_BACKEND": "ipc", "NCCL_NVLS_ENABLE": "0"}, script="mp_late_peer_worker.py")
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert res["timed_out"] == [True, True] and res["recovered_bit_exact"] == [True, True]
    assert res["safe_mode_fallbacks"][0] > 0 and res["safe_mode_fallbacks"] == res["safe_mode_fallbacks"][::-1]
    assert res["replicas_equal"]
