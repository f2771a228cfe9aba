"""Worker for the world_size-2 tests: run under torch.distributed.run.  With `cpu` it exercises the
host-side sharding and collective plumbing over gloo; with `gpu` it runs the data-parallel MLP step."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "pytorch-rs_b200"))
sys.path.insert(0, ROOT)

from torch_rs import distributed as dist  # noqa: E402


def cpu_main(out_path):
    backend = dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    total = 65536 + 3
    begin, end = dist.shard_bounds(total, rank, world)
    covered = dist.all_reduce_host(np.array([end - begin], dtype=np.int64))
    # each rank contributes its slab of a known vector; the sum must equal the full reduction
    vec = np.arange(total, dtype=np.float64)
    partial = np.array([vec[begin:end].sum()])
    summed = dist.all_reduce_host(partial)
    biggest = dist.all_reduce_host(np.array([float(rank)]), op="max")
    # the collective's C entry points refuse bad arguments on the host, before any NCCL or CUDA call
    import ctypes
    from torch_rs import _abi, _host
    lib = _abi.lib()
    comm = ctypes.c_void_p()
    refused = [lib.trs_comm_init_rank(0, world, world, b"\0" * 128, ctypes.byref(comm)),     # rank outside the job
               lib.trs_comm_init_rank(-1, world, rank, b"\0" * 128, ctypes.byref(comm)),     # no such device
               lib.trs_comm_allreduce_sum_f32(None, None, 16, None)]                          # no communicator
    size = ctypes.c_int32(-1)
    _host.check(_host.lib().trsh_comm_size(ctypes.byref(size)))                               # gloo only: no engine communicator
    dist.all_reduce_gradients([])                                                             # nothing to do, must not raise
    all_refused = dist.all_reduce_host(np.array([float(all(r == 1 for r in refused) and size.value == 1)]), op="sum")
    dist.barrier()
    if rank == 0:
        json.dump({"backend": backend, "world": world, "covered": int(covered[0]), "total": total,
                   "sum": float(summed[0]), "expected_sum": float(vec.sum()), "max_rank": float(biggest[0]), "ranks_refusing_bad_arguments": float(all_refused[0]),
                   "local_rank": dist.get_node_local_rank()}, open(out_path, "w"))
    dist.destroy_process_group()


def gpu_main(out_path):
    """Data-parallel MLP step: rows of X sharded, W1/W2/b1 replicated, gradients all-reduced; rank 0
    compares the result with the single-GPU step over the whole batch."""
    import torch_rs as torch
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = f"cuda:{dist.get_node_local_rank()}"
    rng = np.random.default_rng(0)
    bsz, d, h, o = 1024, 256, 512, 128
    xs = rng.standard_normal((bsz, d)).astype(np.float32)
    w1 = (rng.standard_normal((d, h)) / 16).astype(np.float32)
    w2 = (rng.standard_normal((h, o)) / 16).astype(np.float32)
    b1 = (0.1 * rng.standard_normal(h)).astype(np.float32)

    def step(rows):
        X = torch.tensor(xs[rows], device=dev)
        W1, W2 = torch.tensor(w1, device=dev, requires_grad=True), torch.tensor(w2, device=dev, requires_grad=True)
        B1 = torch.tensor(b1, device=dev, requires_grad=True)
        loss = (torch.relu(X @ W1 + B1) @ W2).sum()
        loss.backward()
        return loss, (W1, W2, B1)

    begin, end = dist.shard_bounds(bsz, rank, world)
    # several steps back to back: each exchange runs on the side stream under the next kernels, so a missing
    # ordering would show as a step whose gradients differ from the first one's
    history = []
    for _ in range(4):
        loss, params = step(slice(begin, end))
        dist.all_reduce_gradients(params)
        history.append([p.grad.numpy() for p in params])
    repeatable = all(np.array_equal(a.view(np.uint32), b.view(np.uint32)) for later in history[1:] for a, b in zip(history[0], later))
    total_loss = dist.all_reduce_host(np.array([loss.item()], dtype=np.float64))[0]
    grads = history[-1]
    # one tensor summed in place over the ranks, and a value derived from it afterwards
    t = torch.tensor(np.full((3, 5), float(rank + 1), dtype=np.float32), device=dev)
    dist.all_reduce_(t)
    summed_ok = bool(np.array_equal((t * 2.0).numpy(), np.full((3, 5), 2.0 * sum(range(1, world + 1)), dtype=np.float32)))
    if rank == 0:
        full_loss, full_params = step(slice(0, bsz))
        worst = 0.0
        for g, p in zip(grads, full_params):
            want = p.grad.numpy().astype(np.float64)
            rms = np.sqrt(np.mean(want ** 2))
            worst = max(worst, float(np.max(np.abs(g - want) / (1e-5 * np.sqrt(bsz) * np.maximum(np.abs(want), rms) + 1e-30))))
        json.dump({"world": world, "worst_error_over_bound": worst, "loss": float(total_loss), "full_loss": float(full_loss.item()),
                   "repeatable": bool(repeatable), "all_reduce_in_place_ok": summed_ok},
                  open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    {"cpu": cpu_main, "gpu": gpu_main}[sys.argv[1]](sys.argv[2])
