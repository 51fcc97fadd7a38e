"""Headline benchmark: ResNet-50 data-parallel training with compressed gradients.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                      (the reference arm)

Config (weak scaling): ResNet-50, batch 256 per GPU, 224x224x3 synthetic images,
1000 classes, random init, bf16 autocast with fp32 gradients, 25 MB DDP buckets,
every bucket all-reduced by the fused compressed kernel at 8 bits/value, fused
SGD. ``value`` is total images/s over all GPUs for K steps with device-resident
inputs (CUDA events, max over ranks); ``e2e`` is the same K steps through
``Trainer.step`` with each step's uint8 batch copied from pinned host memory and
the loss read back. Inputs plus activations exceed the 126 MB L2 by far, so no
L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import time

import torch
import torch.distributed as dist

METRIC = "train samples/s (ResNet-50 DDP, compressed gradient all-reduce at 8 bit/value)"


class _SmiClocks:
    """nvidia-smi poller for the reference arm (which imports nothing of gcow_b200): SM clock and
    throttle reasons every 200 ms while the timed region runs."""
    _Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        import threading
        self.gpu, self.rows, self._stop = gpu, [], threading.Event()
        self._th = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        import subprocess
        while not self._stop.is_set():
            try:
                txt = subprocess.run(["nvidia-smi", f"--query-gpu={self._Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu)], capture_output=True, text=True, timeout=10).stdout
                f = [x.strip() for x in txt.strip().splitlines()[0].split(",")]
                self.rows.append((float(f[0]), float(f[1]), f[2:6]))
            except Exception:  # noqa: BLE001 - a missing or slow nvidia-smi only loses a sample
                pass
            self._stop.wait(0.2)

    def start(self):
        self._th.start()
        return self

    def stop(self):
        import statistics
        self._stop.set()
        self._th.join(timeout=15)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[0] for r in self.rows), "sm_max_mhz": max(r[1] for r in self.rows),
                "reasons": reasons, "samples": len(self.rows)}


def reference_arm(args) -> int:
    """The reference's own ImageNet training step, unmodified.

    ``baseline/build_ref.sh`` puts three things under ``baseline/_ref``: the
    reference's CPU codec (sw/src/*.c) as a shared library and byte-for-byte
    copies of hw/models/*.py. The scripts import ``zfpy``, which this image does
    not have; ``baseline/zfpy.py`` provides the two calls they make on top of the
    reference's own codec library. This arm then does what the reference's
    ``main_worker`` does (hw/models/train_imagenet.py:199-253: torchvision
    ``resnet50()``, DistributedDataParallel when there is more than one rank,
    ``CrossEntropyLoss``, ``SGD(lr, momentum, weight_decay)``) and calls the
    reference's ``train()`` (hw/models/train_imagenet.py:404-486) on a list of
    pinned host batches with ``zfp_mode='rate'`` and 8 bits per value. The
    step is host-synchronous (the gradient goes to the host, through the CPU
    codec and back), so the wall clock between two synchronisations is the
    end-to-end time; fp32 compute, because the reference has no autocast.
    Nothing of gcow_b200 is imported on this path."""
    import types
    here = os.path.dirname(os.path.abspath(__file__))
    ref_dir = os.path.join(here, "baseline", "_ref")
    if not (os.path.exists(os.path.join(ref_dir, "libgcowref.so"))
            and os.path.exists(os.path.join(ref_dir, "models", "train_imagenet.py"))):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref is empty: run baseline/build_ref.sh with a reference checkout"}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    sys.path.insert(0, os.path.join(here, "baseline"))            # zfpy stand-in
    sys.path.insert(0, os.path.join(ref_dir, "models"))
    try:
        import train_imagenet as ref
    except Exception as e:  # noqa: BLE001 - whatever stops the import is the answer
        print(json.dumps({"impl": "reference", "unavailable": f"import of hw/models/train_imagenet.py failed: {e!r}"[:300]}))
        return 0

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29534", __file__] + sys.argv[1:]
        return subprocess.call(cmd)
    warmup, steps = max(args.warmup, 1), args.steps
    try:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        if world > 1:
            dist.init_process_group(backend="nccl", init_method="env://", world_size=world, rank=rank)
        # the reference's defaults (hw/models/train_imagenet.py:36-94) with arch and batch of the headline config
        rargs = types.SimpleNamespace(arch="resnet50", zfp_mode="rate", lr=0.1, momentum=0.9, weight_decay=1e-4,
                                      print_freq=10 ** 9, gpu=local, distributed=world > 1, batch_size=args.batch)
        ref.g_arch, ref.g_mode = rargs.arch, rargs.zfp_mode
        model = ref.models.__dict__[rargs.arch]()
        model.cuda(local)
        if world > 1:
            model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])
        criterion = torch.nn.CrossEntropyLoss().to(device)
        optimizer = torch.optim.SGD(model.parameters(), rargs.lr, momentum=rargs.momentum,
                                    weight_decay=rargs.weight_decay)
        g = torch.Generator().manual_seed(rank)
        pool = [(torch.randn(args.batch, 3, 224, 224, generator=g).pin_memory(),
                 torch.randint(0, 1000, (args.batch,), generator=g).pin_memory()) for _ in range(2)]
        nparam = sum(p.numel() for p in model.parameters())

        def run(n):
            batches = [pool[i % len(pool)] for i in range(n)]
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            with contextlib.redirect_stdout(sys.stderr):      # the script prints its progress meters; keep stdout for the JSON line
                diverged = ref.train(int(args.rate), batches, model, criterion, optimizer, 0, device, rargs)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([dt], device=device, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt = float(t[0])
            return dt, diverged

        run(warmup)
        codec0, xfer0 = ref.g_total_codec_sec, ref.g_total_transfer_sec
        sampler = None
        if rank == 0:
            sampler = _SmiClocks(local).start()
        sec, diverged = run(steps)
        clocks = sampler.stop() if sampler else None
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference train() failed: {e!r}"[:300]}))
        return 0
    if rank == 0:
        total = args.batch * world
        v = total * steps / sec
        img_bytes = args.batch * 3 * 224 * 224 * 4 + args.batch * 8
        print(json.dumps({
            "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": sec * 1e3 / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32 (the reference has no autocast)", "impl": "reference",
            "data": "synthetic (random fp32 images / labels in pinned host memory, random-init weights)",
            "config": {"model": "resnet50 (torchvision, as hw/models/train_imagenet.py builds it)", "global_batch": total,
                       "per_gpu_batch": args.batch, "image": 224, "parallelism": f"dp{world}",
                       "rate_bits_per_value": int(args.rate), "zfp_mode": "rate",
                       "codec": "reference sw/src/*.c on the host CPU behind the zfpy calls of the script",
                       "timing": "host clock around the reference's train() between two device synchronisations, max over ranks"},
            "e2e": {"value": v, "unit": "images/s", "ms_per_step": sec * 1e3 / steps,
                    "h2d_bytes_per_step": img_bytes + 4 * nparam, "d2h_bytes_per_step": 4 * nparam + 12},
            "codec_sec_per_step": (ref.g_total_codec_sec - codec0) / steps,
            "transfer_sec_per_step": (ref.g_total_transfer_sec - xfer0) / steps,
            "gpu_launches": 0, "clocks": clocks, "diverged": bool(diverged)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def timed_steps(fn, steps: int):
    """K calls of fn bracketed by barrier + synchronize; device time via CUDA events, max over ranks."""
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    dist.barrier()
    ms = torch.tensor([a.elapsed_time(b), wall * 1e3], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms[0]), float(ms[1])


def nccl_arm(args, device, loader, kind) -> float:
    """Samples/s of the uncompressed baseline (PyTorch ops, NCCL fp32 gradient all-reduce), device-timed like the
    main arm, for the same number of steps."""
    from gcow_b200.config import GcowConfig
    from gcow_b200.train import Trainer
    cfg = GcowConfig.from_env(variant="nccl", timeout_ms=20000)
    tr = Trainer(args.model, batch_size=args.batch, cfg=cfg, ops="torch", seq_len=args.seq_len, device=device)
    pool = []
    for _ in range(4):
        inp, tgt = loader.next()
        pool.append((inp.to(device), tgt.to(device)) if kind == "resnet" else tuple(t.to(device) for t in inp))
    it = {"i": 0}

    def step():
        tr.step_device(pool[it["i"] % len(pool)])
        it["i"] += 1
    for _ in range(3):
        step()
    ms, _ = timed_steps(step, args.steps)
    del tr, pool
    torch.cuda.empty_cache()
    return args.batch * dist.get_world_size() * args.steps / (ms / 1e3)


def side_metrics(device, rank, world) -> dict:
    """The two other headline metrics, measured in this process after the training loops: the stand-alone codec
    (256 MB fp32, 8 bit/value) and, on more than one GPU, the fused all-reduce of a 256 MB buffer at 4/8/16
    bit/value against ``dist.all_reduce`` plus a 1 M-value bit-exactness check against the host model."""
    import numpy as np
    import gcow_b200 as g
    from gcow_b200.codec import ZfpParams
    from gcow_b200.comm import CompressedAllReduce
    from gcow_b200.comm.oracle import allreduce_oracle
    from gcow_b200.config import GcowConfig
    from gcow_b200.bench.allreduce_sweep import time_calls
    out = {}
    n = 64 << 20
    gen = torch.Generator(device=device).manual_seed(rank)
    x = torch.randn(n, device=device, generator=gen) * 1e-3
    p8 = ZfpParams.from_rate(8, 1)
    c = g.compress(x, params=p8)
    y = torch.empty_like(x)
    enc = time_calls(lambda: g.compress(x, params=p8), 10, warmup=50)
    dec = time_calls(lambda: g.decompress(c, out=y), 10, warmup=50)
    out["codec_rate8_256MB"] = {"enc_ms": enc, "dec_ms": dec, "enc_gbs": n * 4 / enc / 1e6, "dec_gbs": n * 4 / dec / 1e6,
                                "max_abs_err": float((x - y).abs().max())}
    del c, y
    if world > 1:
        bufs = [x, x.clone()]
        k = {"i": 0}

        def nccl():
            dist.all_reduce(bufs[k["i"] & 1])
            k["i"] += 1
        out["allreduce_256MB_ms"] = {"nccl_fp32": time_calls(nccl, 10, warmup=50)}
        exact = True
        for rate in (4, 8, 16):
            cfg = GcowConfig(rate=rate, comm_ctas=4096, timeout_ms=20000, average=True)
            ar = CompressedAllReduce(n, cfg, device=device)
            for t in bufs:      # fresh N(0, 1e-3) values for every rate: the output of a coarser rate is low-entropy data,
                t.normal_(generator=gen).mul_(1e-3)   # which leaves the coder's fast path and would time something else

            def fused():
                ar(bufs[k["i"] & 1])
                k["i"] += 1
            # the host-side check of the previous rate left the GPU idle and its clocks low: 100 calls bring them back
            out["allreduce_256MB_ms"][f"fused_rate{rate}"] = time_calls(fused, 10, warmup=100)
            ar.check()
            # bit-exactness on 1 M values: every rank gathers all inputs and runs the host model
            m = 1 << 20
            xin = torch.randn(m, device=device, generator=gen) * 1e-3
            allx = [torch.empty_like(xin) for _ in range(world)]
            dist.all_gather(allx, xin)
            res = ar(xin.clone(), variant="twoshot")
            ar.check()
            want = allreduce_oracle(np.stack([t.cpu().numpy() for t in allx]), ar.params, "twoshot",
                                    shift=ar._avg_shift)
            if ar._avg_scale != 1.0:
                want = want * np.float32(ar._avg_scale)
            ok = torch.tensor([int(np.array_equal(res.cpu().numpy().view(np.uint32), want.view(np.uint32)))],
                              device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            exact = exact and bool(int(ok[0]))
            del ar
        out["allreduce_bitexact"] = exact
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="gcow", choices=["gcow", "reference", "nccl"])
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: 256 images for a ResNet, 32 sequences for BERT)")
    ap.add_argument("--rate", type=float, default=8.0)
    ap.add_argument("--ops", default="own", choices=["own", "torch"])
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--comm-ctas", type=int, default=0,
                    help="CTAs of the fused all-reduce (0: 148 for ResNet, 296 for BERT, whose 1.3 GB of gradients per step "
                         "make the collective itself worth more SM time)")
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the NCCL arm and the codec / all-reduce side measurements after the timed loops")
    args = ap.parse_args()
    args.batch = args.batch or (32 if args.model.replace("-", "_").startswith("bert") else 256)
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    if args.gpus > 1 and "RANK" not in os.environ:
        # convenience: re-launch under torchrun
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", __file__] + sys.argv[1:]
        return subprocess.call(cmd)

    from gcow_b200.config import GcowConfig
    from gcow_b200.train import Trainer, make_loader
    from gcow_b200.utils.tracing import ClockSampler

    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    variant = "nccl" if args.impl == "nccl" else args.variant
    comm_ctas = args.comm_ctas or (296 if args.model.startswith("bert") else 148)
    cfg = GcowConfig.from_env(rate=args.rate, variant=variant, comm_ctas=comm_ctas, timeout_ms=20000)
    tr = Trainer(args.model, batch_size=args.batch, cfg=cfg, ops=args.ops if args.impl != "nccl" else "torch",
                 seq_len=args.seq_len, device=device)
    rank, world = tr.rank, tr.world
    loader = make_loader(tr.kind, args.batch, args.seq_len, seed=rank)

    # device-resident copies of the pool for the kernel-only loop
    pool = []
    for _ in range(4):
        inp, tgt = loader.next()
        if tr.kind == "resnet":
            pool.append((inp.to(device), tgt.to(device)))
        else:
            pool.append(tuple(t.to(device) for t in inp))
    it = {"i": 0}

    def dev_step():
        tr.step_device(pool[it["i"] % len(pool)])
        it["i"] += 1

    nxt = {"b": loader.next()}

    def e2e_step():
        # this step's batch was staged by the previous call; the next one is copied while this step computes
        cur, nxt["b"] = nxt["b"], loader.next()
        tr.step(cur[0], cur[1], prefetch=nxt["b"])

    for _ in range(args.warmup):
        dev_step()
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    # which kernel family served each convolution call of one step (forward pass of every layer)
    from gcow_b200.ops import kernels as _kern
    _kern.conv_path_counts(reset=True)
    dev_step()
    torch.cuda.synchronize()
    conv_paths = _kern.conv_path_counts(reset=True)

    sampler = ClockSampler(local).start() if rank == 0 else None
    l0 = tr.gpu_launches()
    dev_ms, _ = timed_steps(dev_step, args.steps)
    launches = tr.gpu_launches() - l0
    h0, d0 = tr.h2d_bytes, tr.d2h_bytes
    e2e_ms, e2e_wall = timed_steps(e2e_step, args.steps)
    h2d = (tr.h2d_bytes - h0) // args.steps
    d2h = (tr.d2h_bytes - d0) // args.steps
    clocks = sampler.stop() if sampler else None
    final_loss = tr.last_loss()

    # ---- same box, same process: the uncompressed NCCL(+cuBLAS/cuDNN) arm and the two other headline metrics
    nccl_value = None
    extra = {}
    if args.impl == "gcow" and not args.no_extra:
        try:
            nccl_value = nccl_arm(args, device, loader, tr.kind)
        except Exception as e:  # noqa: BLE001 - the side measurements must not lose the headline line
            extra["nccl_arm_error"] = repr(e)[:200]
        try:
            extra.update(side_metrics(device, rank, world))
        except Exception as e:  # noqa: BLE001
            extra["error"] = repr(e)[:200]
    from gcow_b200.ops import kernels as _k
    kernel_errors = int(_k.check_errors(raise_on_error=False))

    if rank == 0:
        total = args.batch * world
        unit = "images/s" if tr.kind == "resnet" else "sequences/s"
        out = {
            "metric": METRIC if args.model == "resnet50" else f"train samples/s ({args.model})",
            "value": total * args.steps / (dev_ms / 1e3), "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (total * args.steps / (dev_ms / 1e3)) / nccl_value if nccl_value else None,
            "baseline": {"what": "the reference publishes no number; this is the uncompressed NCCL(+cuBLAS/cuDNN) DDP arm "
                                 "(--impl nccl) timed in this process for the same steps", "value": nccl_value},
            "dtype": "bf16",
            "data": "synthetic (random uint8 images / labels, random-init weights)",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": total, "per_gpu_batch": args.batch,
                       "seq_len": args.seq_len if tr.kind == "bert" else None, "image": 224,
                       "parallelism": f"dp{world}", "bucket_mb": cfg.bucket_mb, "rate_bits_per_value": args.rate,
                       "variant": cfg.variant, "ops": args.ops, "comm_ctas": tr.hook_state.ar.ctas if tr.hook_state else 0,
                       "conv_paths_per_step": conv_paths,
                       "conv_backend": {"own": sum(v for k, v in conv_paths.items() if k != "cudnn"),
                                        "cudnn": conv_paths.get("cudnn", 0)},
                       "attention": ("fused tcgen05" if tr.kind == "bert" and args.ops == "own" else None),
                       "l2": "inputs+activations larger than L2, no flush"},
            "e2e": {"value": total * args.steps / (e2e_ms / 1e3), "unit": unit, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "final_loss": final_loss,
            "kernel_error_word": kernel_errors,
            "extra": extra,
        }
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
