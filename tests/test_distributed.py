"""Multi-process paths: world_size-2 over gloo on CPU (sharding + collective plumbing), and the
data-parallel MLP step on 2 GPUs over NCCL (skipped unless two devices are visible)."""
import json
import os
import socket
import subprocess
import sys

import pytest

from torch_rs import distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(mode, tmp_path, nproc=2):
    out = tmp_path / "result.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "dist_worker.py"), mode, str(out)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    return json.load(open(out))


def test_shard_bounds_cover_exactly_once():
    for total in (0, 1, 7, 64, 65536, 65539):
        for world in (1, 2, 3, 4, 8):
            spans = [dist.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dist.shard_bounds(10, 2, 2)


def test_local_rank_convention(monkeypatch):
    monkeypatch.setenv("LOCAL_RANK", "3")
    assert dist.get_node_local_rank() == 3
    monkeypatch.delenv("LOCAL_RANK")
    assert dist.get_node_local_rank(fallback_rank=1) == 1
    with pytest.raises(RuntimeError):
        dist.get_node_local_rank()


def test_world_size_two_gloo_sharding_and_collectives(tmp_path):
    r = launch("cpu", tmp_path)
    assert r["backend"] == "gloo" and r["world"] == 2
    assert r["covered"] == r["total"]
    assert r["sum"] == r["expected_sum"]
    assert r["max_rank"] == 1.0 and r["local_rank"] == 0
    assert r["ranks_refusing_bad_arguments"] == 2.0


@pytest.mark.gpu
def test_data_parallel_mlp_gradients_match_single_gpu(tmp_path):
    import torch_rs as torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    r = launch("gpu", tmp_path)
    assert r["world"] == 2
    assert r["worst_error_over_bound"] <= 1.0
    assert r["repeatable"] and r["all_reduce_in_place_ok"]
    assert abs(r["loss"] - r["full_loss"]) <= 1e-4 * abs(r["full_loss"]) + 1e-3


def test_cpu_list_parsing_and_numa_binding_without_a_device():
    assert dist._parse_cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert dist._parse_cpu_list("") == set()
    import torch_rs as torch
    if not torch.cuda.is_available():
        before = os.sched_getaffinity(0)
        assert dist.bind_to_device_numa_node(0) is None          # no device: nothing is changed
        assert os.sched_getaffinity(0) == before
