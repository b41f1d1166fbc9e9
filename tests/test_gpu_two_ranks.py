"""Token-sharded projection set on two GPUs over NCCL (skipped when fewer than two are visible):
each rank runs one training-step projection set on its shard; after the step every rank must hold
the same dW buckets, and they must equal the sum of the two shards' un-reduced buckets computed
by a single process."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOKENS_PER_RANK = 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _small_shape(entry):
    entry.load_package()
    from nanogpt_120a_b200.projection_set import ModelShape

    return ModelShape("tiny-proj-set", 2, 128, 256, 512)


def _rank(rank, world, port, out_dir, use_cpp_step=False, reproducible=False):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import __graft_entry__ as entry

    shape = _small_shape(entry)
    from nanogpt_120a_b200.projection_set import ProjectionSet

    extra = dict(total_tokens=world * TOKENS_PER_RANK, reproducible_sharding=True, input_seed_offset=0) if reproducible else {}
    ps = ProjectionSet(shape, TOKENS_PER_RANK, dev, seed=77, token_offset=rank * TOKENS_PER_RANK,
                       process_group=None if use_cpp_step else dist.group.WORLD, **extra)
    if reproducible:  # this rank's rows of one global batch
        whole = ProjectionSet(shape, world * TOKENS_PER_RANK, dev, seed=77)
        rows = slice(rank * TOKENS_PER_RANK, (rank + 1) * TOKENS_PER_RANK)
        ps.x = {w: t[rows].contiguous() for w, t in whole.x.items()}
        ps.dy = {w: t[rows].contiguous() for w, t in whole.dy.items()}
        del whole
    if use_cpp_step:
        from nanogpt_120a_b200.host_step import HostStep

        host = HostStep(ps, process_group=dist.group.WORLD)  # the driver's own NCCL communicator
        host.step()
        torch.cuda.synchronize()
        buckets = [b.cpu() for b in host.buckets]
        host.close()
    else:
        ps.step()
        torch.cuda.synchronize()
        buckets = [b.cpu() for b in ps.buckets]
    torch.save(buckets, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_step_reduces_dw(tmp_path):
    import torch.multiprocessing as mp

    import __graft_entry__ as entry

    port = _free_port()
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    for a, b in zip(*got):
        assert torch.equal(a, b)  # all-reduce leaves identical buckets on both ranks

    # single process: the same two shards, no process group, buckets summed on the host
    shape = _small_shape(entry)
    from nanogpt_120a_b200.projection_set import ProjectionSet

    dev = torch.device("cuda:0")
    total = None
    for r in range(2):
        ps = ProjectionSet(shape, TOKENS_PER_RANK, dev, seed=77, token_offset=r * TOKENS_PER_RANK)
        ps.step()
        torch.cuda.synchronize()
        shard = [b.cpu().double() for b in ps.buckets]
        total = shard if total is None else [t + s for t, s in zip(total, shard)]
    for want, have in zip(total, got[0]):
        # NCCL adds the two f32 shards once: equal to the f64 sum up to one f32 rounding
        assert torch.allclose(have.double(), want, rtol=1e-6, atol=1e-9)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_cpp_step_equals_python_step(tmp_path):
    """The C++ step driver with its own NCCL communicator (ncclAllReduce issued from C++ on a communication
    stream) leaves the same reduced buckets as the Python set over torch.distributed."""
    import torch.multiprocessing as mp

    port = _free_port()
    (tmp_path / "py").mkdir()
    (tmp_path / "cpp").mkdir()
    mp.spawn(_rank, args=(2, port, str(tmp_path / "py")), nprocs=2, join=True)
    mp.spawn(_rank, args=(2, _free_port(), str(tmp_path / "cpp"), True), nprocs=2, join=True)
    for r in range(2):
        for a, b in zip(torch.load(tmp_path / "py" / f"rank{r}.pt"), torch.load(tmp_path / "cpp" / f"rank{r}.pt")):
            assert torch.equal(a, b)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_reproducible_sharding_matches_one_gpu(tmp_path):
    """Two ranks holding the two halves of one batch, with the step's amaxes all-reduced (max) in one collective
    and the unsharded RNG index spaces: the reduced dW equals the dW of the whole batch on one GPU up to f32
    summation order."""
    import torch.multiprocessing as mp

    import __graft_entry__ as entry

    mp.spawn(_rank, args=(2, _free_port(), str(tmp_path), True, True), nprocs=2, join=True)
    got = torch.load(tmp_path / "rank0.pt")
    shape = _small_shape(entry)
    from nanogpt_120a_b200.projection_set import ProjectionSet

    dev = torch.device("cuda:0")
    ps = ProjectionSet(shape, 2 * TOKENS_PER_RANK, dev, seed=77)
    ps.step()
    torch.cuda.synchronize()
    for want, have in zip(ps.buckets, got):
        rel = (have.double() - want.cpu().double()).norm() / want.cpu().double().norm()
        assert rel <= 1e-6, float(rel)
