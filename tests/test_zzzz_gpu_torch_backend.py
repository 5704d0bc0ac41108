"""The ``torch.distributed`` backend "mccs" and the functional collectives of
``mccs_b200.ops`` on CUDA tensors: ordinary CUDA memory goes through the communicator's
staging arena (copy in, collective in place, copy out, all on the caller's stream), tensors
in service memory are used where they are. Two client processes of a stand-alone daemon; on
a machine with one GPU both sit on cuda:0 (the daemon then runs each collective as one
cooperative launch), with two or more each has its own.

The reference has no framework layer; parity is with what the same calls give on the
``nccl`` backend: the values asserted below.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

from helpers import REPO, write_config

pytestmark = pytest.mark.gpu

COLLECTIVES = r"""
import os, sys, torch, torch.distributed as dist
import mccs_b200 as M
import mccs_b200.process_group as mpg
from mccs_b200 import ops
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); dev = int(os.environ["DEV"])
torch.cuda.set_device(dev)
cuda = torch.device("cuda", dev)
dist.init_process_group("mccs", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=n)
# ordinary CUDA tensors: staged
t = torch.arange(100000, dtype=torch.float32, device=cuda) + rank
dist.all_reduce(t)
assert torch.equal(t, sum(torch.arange(100000, dtype=torch.float32, device=cuda) + r for r in range(n))), "all_reduce f32"
h = (torch.arange(4097, device=cuda) % 7 + rank).to(torch.bfloat16)
dist.all_reduce(h, op=dist.ReduceOp.AVG)
assert torch.allclose(h.float(), (torch.arange(4097, device=cuda) % 7).float() + (n - 1) / 2, atol=0.1), "all_reduce bf16 avg"
m = torch.tensor([float(rank)], device=cuda); dist.all_reduce(m, op=dist.ReduceOp.MAX); assert m.item() == n - 1
b = torch.full((5,), float(rank), device=cuda); dist.broadcast(b, src=1); assert bool(torch.all(b == 1)), "broadcast"
nz = torch.tensor([-0.0, float("nan"), float("-inf"), 1.5], device=cuda) if rank == 0 else torch.ones(4, device=cuda)
dist.broadcast(nz, src=0)
assert nz.view(torch.int32).tolist() == torch.tensor([-0.0, float("nan"), float("-inf"), 1.5]).view(torch.int32).tolist(), "broadcast bits"
sv = torch.zeros(4, 6, device=cuda); col = sv[:, 1:4]
if rank == 1: col.copy_(torch.arange(12., device=cuda).reshape(4, 3))
dist.broadcast(col, src=1)
assert torch.equal(sv[:, 1:4], torch.arange(12., device=cuda).reshape(4, 3)) and float(sv[:, 0].abs().sum()) == 0, "broadcast view"
outs = [torch.empty(3, dtype=torch.int64, device=cuda) for _ in range(n)]
dist.all_gather(outs, torch.full((3,), rank, dtype=torch.int64, device=cuda))
assert all(bool(torch.all(o == r)) for r, o in enumerate(outs)), "all_gather"
big = torch.empty(n * 4, device=cuda); dist.all_gather_into_tensor(big, torch.full((4,), float(rank), device=cuda))
assert torch.equal(big, torch.arange(n, device=cuda).repeat_interleave(4).float()), "all_gather_into_tensor"
rs = torch.empty(2, device=cuda); dist.reduce_scatter_tensor(rs, torch.arange(2 * n, device=cuda).float())
assert torch.equal(rs, torch.arange(2 * n, device=cuda).float().reshape(n, 2)[rank] * n), "reduce_scatter_tensor"
# tensors in service memory: in place, no staging
z, keep = mpg.empty(1 << 20, torch.float32, device=dev)
z.fill_(rank + 1.0); assert mpg.in_service_memory(z) and not mpg.in_service_memory(t)
dist.all_reduce(z); assert bool(torch.all(z == n * (n + 1) / 2)), "all_reduce in service memory"
# a CPU tensor through the same group (staged through the GPU)
c = torch.arange(10, dtype=torch.float32) + rank
dist.all_reduce(c); assert torch.equal(c, sum(torch.arange(10, dtype=torch.float32) + r for r in range(n))), "all_reduce of a CPU tensor"
dist.barrier()
# the functional form on a communicator of its own
comm = M.Communicator(int(os.environ["COMM2"]), rank, n, device=dev)
x = torch.full((3000,), float(rank + 1), device=cuda, dtype=torch.float16)
y = ops.all_reduce(comm, x, op="sum"); torch.cuda.synchronize()
assert y.data_ptr() == x.data_ptr() and bool(torch.all(x == n * (n + 1) / 2)), "ops.all_reduce"
g = torch.empty(n * 1000, device=cuda, dtype=torch.int32)
ops.all_gather(comm, torch.full((1000,), rank, device=cuda, dtype=torch.int32), g); torch.cuda.synchronize()
assert torch.equal(g, torch.arange(n, device=cuda, dtype=torch.int32).repeat_interleave(1000)), "ops.all_gather"
q = comm.query(); assert q["async_error"] == 0 and q["device_error"] == 0
torch.cuda.synchronize()
ops.arena(comm).release(); comm.destroy()
print(f"rank {rank} ok", flush=True)
torch.cuda.synchronize()
mpg.shutdown(); keep.free()
dist.destroy_process_group()
M.finalize()
"""

TORCH_DDP = r"""
import os, sys, torch, torch.distributed as dist
import mccs_b200 as M
import mccs_b200.process_group as mpg
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); dev = int(os.environ["DEV"])
torch.cuda.set_device(dev)
cuda = torch.device("cuda", dev)
dist.init_process_group("mccs", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=n)
torch.manual_seed(0)
model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 8)).to(cuda)
ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev])
x = torch.randn(16, 64, generator=torch.Generator().manual_seed(rank)).to(cuda)
ddp(x).sum().backward()
torch.cuda.synchronize()
flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
# the same gradients from a plain replica: every rank computes every rank's, in fp32
torch.manual_seed(0)
plain = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 8)).to(cuda)
want = None
for r in range(n):
    plain.zero_grad()
    plain(torch.randn(16, 64, generator=torch.Generator().manual_seed(r)).to(cuda)).sum().backward()
    gr = torch.cat([p.grad.reshape(-1) for p in plain.parameters()])
    want = gr.clone() if want is None else want + gr
assert torch.allclose(flat, want / n, rtol=1e-4, atol=1e-5), float((flat - want / n).abs().max())
print(f"rank {rank} ok", flush=True)
torch.cuda.synchronize()
del ddp
mpg.shutdown()
dist.destroy_process_group()
M.finalize()
"""


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(tmp_path, code, comm2):
    from mccs_b200 import daemon
    ngpu = torch.cuda.device_count()
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, wait_timeout_ms=5000)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        assert sp.backend == "cuda"
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE="2", MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000",
                   PORT=str(_free_port()), COMM2=str(comm2))
        procs = [subprocess.Popen([sys.executable, "-c", code], env=dict(env, RANK=str(r), DEV=str(r if ngpu >= 2 else 0)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
        for r, p in enumerate(procs):
            out, err = p.communicate(timeout=300)
            assert p.returncode == 0 and f"rank {r} ok" in out, out[-1000:] + err[-3000:]
    finally:
        sp.stop()


def test_torch_distributed_backend_on_cuda_tensors(tmp_path):
    _run(tmp_path, COLLECTIVES, 7410)


def test_torch_ddp_over_the_backend_on_gpus(tmp_path):
    """torch's own DistributedDataParallel over the backend: the averaged gradients equal the
    mean of the gradients every rank's batch gives on a plain replica."""
    _run(tmp_path, TORCH_DDP, 7411)
