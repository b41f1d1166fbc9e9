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


def _rank(rank, world, port, out_dir):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import __graft_entry__ as entry

    shape = _small_shape(entry)
    from nanogpt_120a_b200.projection_set import ProjectionSet

    ps = ProjectionSet(shape, TOKENS_PER_RANK, dev, seed=77, token_offset=rank * TOKENS_PER_RANK,
                       process_group=dist.group.WORLD)
    ps.step()
    torch.cuda.synchronize()
    torch.save([b.cpu() for b in ps.buckets], os.path.join(out_dir, f"rank{rank}.pt"))
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
