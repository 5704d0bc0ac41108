"""Data-parallel training driver with synthetic data: ResNet-50 / VGG-16 (fp32, batch
64 per GPU, 224x224x3 images ~N(0,1), labels uniform over 1000 classes) and
GPT-2-medium (bf16 parameters and therefore bf16 gradient buckets, batch 8 per GPU, sequence
1024, token ids uniform over the vocabulary; ``--param-dtype fp32`` keeps fp32 parameters under
bf16 autocast instead), random init, SGD. One rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m mccs_b200.parallel.train --model resnet50 --comm-id 300 --steps 30

``--backend mccs`` sends the 25 MB gradient buckets through the service (the job is a
tenant: ``--comm-id`` is its QoS identity), overlapped with backward; ``--backend nccl``
is torch's DistributedDataParallel over NCCL with the same bucket size, the baseline.
The daemon must already run (``MCCS_CONTROL``), or ``--start-daemon`` lets local rank 0
host it. Prints one JSON line with images/s or tokens/s. ``--save`` / ``--resume`` write and
read a plain ``torch.save`` checkpoint of model and optimizer.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

# One hardware queue per CUDA stream where possible, so that a stream that waits for a
# collective cannot hold up the compute stream (must be set before CUDA initialises).
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--backend", default="mccs", choices=["mccs", "nccl", "none"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--comm-id", type=int, default=300)
    ap.add_argument("--start-daemon", action="store_true")
    ap.add_argument("--control", default="")
    ap.add_argument("--devices", default="", help="comma separated GPU index per rank (default: local rank)")
    ap.add_argument("--name", default="")
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--param-dtype", default="auto", choices=["auto", "fp32", "bf16"],
                    help="parameter (and gradient bucket) type; auto = bf16 for the language model, fp32 for the CNNs")
    ap.add_argument("--comm-ctas", type=int, default=0,
                    help="cap the CTAs of this job's collective kernels (a QoS quota set through the admin "
                         "endpoint), leaving the other SMs to backward; 0 = the planner's choice")
    ap.add_argument("--admin-port", type=int, default=0, help="admin port of a daemon that is already running")
    ap.add_argument("--shard-optimizer", action="store_true",
                    help="ZeRO stage 1 over the service's ReduceScatter: reduce-scattered gradients, 1/n of the optimizer "
                         "state per rank, updated parameters all-gathered (mccs backend; not with --save/--resume)")
    ap.add_argument("--sync-dir", default="", help="co-located jobs: directory in which every job drops '<name>.ready' after its "
                    "warm-up; the timed steps start when --sync-jobs such files exist, so that the jobs' timed regions overlap")
    ap.add_argument("--sync-jobs", type=int, default=0)
    ap.add_argument("--save", default="", help="after the run rank 0 writes model + optimizer state here (torch.save)")
    ap.add_argument("--resume", default="", help="load model + optimizer state written by --save before training")
    args = ap.parse_args()

    from mccs_b200 import models
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    dev_index = int(args.devices.split(",")[rank]) if args.devices else local_rank
    device = torch.device(f"cuda:{dev_index}" if cuda else "cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", device_id=device if cuda else None)

    def barrier():
        if world > 1:
            dist.barrier()

    lm = models.is_language_model(args.model)
    batch = args.batch or (8 if lm else 64)
    torch.manual_seed(1234)          # identical initial weights on every rank
    model = models.build(args.model).to(device)
    bf16_params = args.param_dtype == "bf16" or (args.param_dtype == "auto" and lm and cuda)
    if bf16_params:
        model.to(torch.bfloat16)      # gradients, and with them the buckets that are all-reduced, are bf16
    if cuda and not lm:
        model.to(memory_format=torch.channels_last)   # before gradient buckets are laid out
    model.train()
    opt = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=0.9)
    start_step = 0
    if args.resume:
        # The service keeps no state of its own (neither does the reference's): a job's
        # checkpoint is its model and optimizer, restored before the gradient buckets
        # are laid out over the parameters.
        ck = torch.load(args.resume, map_location=device)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["optimizer"])
        start_step = int(ck.get("step", 0))

    M = None
    ddp = None
    if args.backend == "mccs":
        import mccs_b200 as M
        prefix = args.control or f"/tmp/mccs-train-{os.getuid()}-{os.environ.get('MASTER_PORT', '0')}"
        spawned = None
        if args.start_daemon and local_rank == 0:
            # a stand-alone daemon: every rank is an outside client, nobody blocks on the host
            os.makedirs(prefix, exist_ok=True)
            with open(prefix + "/mccs.toml", "w") as f:
                f.write(M.daemon.default_config(prefix, listen_port=-1))
            spawned = M.daemon.spawn(prefix + "/mccs.toml")
        admin_port = spawned.admin_port if spawned is not None else args.admin_port
        if args.comm_ctas > 0 and local_rank == 0:
            if not admin_port:
                raise SystemExit("--comm-ctas needs --start-daemon or --admin-port")
            rep = M.admin_request(admin_port, {"cmd": "qos_set", "tenants": {str(args.comm_id): {"weight": 1.0, "cta_quota": args.comm_ctas}}})
            assert rep.get("status") == "ok", rep
        barrier()
        if args.start_daemon or args.control:
            M.init(prefix + "/control.sock" if not prefix.endswith(".sock") else prefix)
        comm = M.Communicator(args.comm_id, rank, world, device=dev_index if cuda else rank)
        from mccs_b200.parallel import DataParallel, ShardedDataParallel
        if args.shard_optimizer:
            if args.save or args.resume:
                raise SystemExit("--shard-optimizer keeps 1/n of the optimizer state per rank: no --save/--resume")
            ddp = ShardedDataParallel(model, comm, bucket_mb=args.bucket_mb, broadcast_parameters=world > 1)
            opt = ddp.make_optimizer(torch.optim.SGD, lr=args.lr, momentum=0.9)
        else:
            ddp = DataParallel(model, comm, bucket_mb=args.bucket_mb, broadcast_parameters=world > 1)
        fwd = model
    elif args.backend == "nccl" and world > 1:
        fwd = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev_index] if cuda else None,
                                                        bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
    else:
        fwd = model

    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    if lm:
        vocab = model.cfg.vocab_size
        seq = min(args.seq, model.cfg.max_seq)
        ids = torch.randint(0, vocab, (batch, seq + 1), generator=g).to(device)
        inputs, targets = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        units = batch * seq
    else:
        inputs = torch.randn(batch, 3, 224, 224, generator=g).to(device)
        targets = torch.randint(0, 1000, (batch,), generator=g).to(device)
        units = batch
        if cuda:
            inputs = inputs.contiguous(memory_format=torch.channels_last)

    def step() -> torch.Tensor:
        if ddp is not None:
            ddp.zero_grad()
        else:
            opt.zero_grad(set_to_none=False)
        if lm:
            with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=cuda and not bf16_params):
                loss = fwd(inputs, targets)
        else:
            loss = torch.nn.functional.cross_entropy(fwd(inputs.to(torch.bfloat16) if bf16_params else inputs), targets)
        loss.backward()
        if ddp is not None:
            ddp.finish()
        if args.shard_optimizer and ddp is not None:
            ddp.step(opt)
        else:
            opt.step()
        return loss

    losses = []
    for _ in range(args.warmup):
        losses.append(float(step()))
    if cuda:
        torch.cuda.synchronize()
    barrier()
    if args.sync_dir and args.sync_jobs > 1:
        os.makedirs(args.sync_dir, exist_ok=True)
        if rank == 0:
            open(os.path.join(args.sync_dir, (args.name or args.model) + ".ready"), "w").close()
        deadline = time.time() + 300
        while len([f for f in os.listdir(args.sync_dir) if f.endswith(".ready")]) < args.sync_jobs and time.time() < deadline:
            time.sleep(0.005)
        barrier()
    t0 = time.perf_counter()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for _ in range(args.steps):
        loss = step()
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
    losses.append(float(loss))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        out = {"name": args.name or args.model, "model": args.model, "backend": args.backend, "n_gpus": world,
               "batch_per_gpu": batch, "ms_per_step": ms, "param_dtype": "bf16" if bf16_params else "fp32",
               ("tokens_per_s" if lm else "images_per_s"): units * world / ms * 1e3,
               "first_loss": losses[0] if losses else None, "last_loss": losses[-1],
               "grad_bytes": ddp.gradient_bytes() if ddp is not None else sum(p.numel() * p.element_size() for p in model.parameters()),
               "buckets": len(ddp.buckets) if ddp is not None else None,
               "step": start_step + args.warmup + args.steps}
        if args.save:
            torch.save({"model": model.state_dict(), "optimizer": opt.state_dict(), "step": out["step"]}, args.save)
        print(json.dumps(out), flush=True)
    barrier()
    if ddp is not None:
        ddp.release()
        comm.destroy()
        M.finalize()
        barrier()
        if spawned is not None:
            spawned.stop()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
