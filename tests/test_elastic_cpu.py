"""Failure detection on the host: gloo ranks on CPU, failures made by a rank that
leaves or raises between steps. No GPU is involved."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, tmp_path, nproc=3):
    out = str(tmp_path / "hb")
    env = dict(os.environ, GCOW_HB_MODE=mode, GCOW_TEST_OUT=out, MASTER_ADDR="127.0.0.1")
    port = 29700 + os.getpid() % 200 + (7 if mode == "leave" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_heartbeat_worker.py")]
    subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=180)
    return [json.load(open(f"{out}.{r}")) for r in range(nproc) if os.path.exists(f"{out}.{r}")]


def test_rank_that_leaves_is_detected_by_heartbeat(tmp_path):
    res = _run("leave", tmp_path)
    assert len(res) == 3
    survivors = [r for r in res if not r.get("left")]
    assert len(survivors) == 2
    for r in survivors:
        # either this rank saw rank 2's beat stop, or the other survivor saw it first and posted the abort
        assert r["outcome"] == "restart" and ("2" in r["why"] or "abort posted" in r["why"]), r
        assert r["seconds"] < 30 and r["steps"] >= 3          # noticed within seconds, not at step 200
    assert any("2" in r["why"] for r in survivors)


def test_local_failure_is_broadcast_as_abort(tmp_path):
    res = _run("raise", tmp_path)
    assert len(res) == 3
    assert all(r["outcome"] == "restart" for r in res)
    others = [r for r in res if r["rank"] != 1]
    assert all("abort posted" in r["why"] or "1" in r["why"] for r in others)


def test_reference_launch_flags_map_to_ranks():
    """--world-size / --rank / --dist-url / --gpu / --multiprocessing-distributed of the reference script
    (hw/models/train_imagenet.py:60-94,139-147) become the RANK / WORLD_SIZE / MASTER_* environment."""
    from gcow_b200 import train_cli
    a = train_cli.parse(["--dummy", "--world-size", "2", "--rank", "1", "--dist-url", "tcp://10.0.0.5:4567",
                         "--multiprocessing-distributed", "-j", "8", "--dist-backend", "nccl"])
    env = train_cli.launch_env(a, ngpus=8, local=3)
    assert env == {"RANK": "11", "LOCAL_RANK": "3", "WORLD_SIZE": "16", "MASTER_ADDR": "10.0.0.5", "MASTER_PORT": "4567"}
    b = train_cli.parse(["--dummy", "--world-size", "4", "--rank", "2", "--gpu", "1"])
    env = train_cli.launch_env(b, ngpus=8)
    assert env["RANK"] == "2" and env["WORLD_SIZE"] == "4" and env["LOCAL_RANK"] == "1" and env["MASTER_ADDR"] == "127.0.0.1"
    # --pretrained is accepted; without the weights in the local hub cache the model builder says so
    from gcow_b200.models import build_model
    with pytest.raises((RuntimeError, KeyError)):
        build_model("resnet18", pretrained=True)


@pytest.mark.parametrize("failing", ["", "1", "0,2"])
def test_safe_mode_redo_is_agreed_across_ranks(failing):
    """The fused collective can time out on some ranks only. finish_step must then redo the step's buckets with the
    plain all-reduce on EVERY rank (or on none), from the untouched local gradients, so the replicas stay equal and
    no rank is left alone inside a collective."""
    env = dict(os.environ, FAILING=failing, MASTER_ADDR="127.0.0.1")
    port = 29450 + os.getpid() % 200 + len(failing)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_agree_worker.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=180)
    assert p.returncode == 0 and p.stdout.count("ok") == 3, p.stdout[-1500:] + p.stderr[-1500:]
