"""Token-sharded path on two CPU ranks over gloo: shard plan, MS-EDEN index-space offsets, the
shared global scale (all-reduce max), the per-layer dW bucket all-reduce (sum), and host-side
failure detection (a rank that never joins the collective).  The per-rank arithmetic is done
by the CPU oracle, so the test exercises exactly the host logic the GPU ranks run."""
import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIGN, SCALE = 0x12345678, 0x9ABCDEF0
TOKENS, IN_DIM, OUT_DIM = 256, 64, 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup(rank, world, port, timeout_s=60):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    import __graft_entry__ as entry
    from oracle import oracle

    entry.load_package()
    from nanogpt_120a_b200 import sharding

    return oracle, sharding


def _data():
    from helpers import normal

    x = torch.from_numpy(normal(1, (TOKENS, IN_DIM)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    dy = torch.from_numpy(normal(2, (TOKENS, OUT_DIM), 1e-3).astype(np.float32)).to(torch.bfloat16).float().numpy()
    return x, dy


def _shard_dw(oracle, x, dy, gs_e, first_token, out_dim, in_dim):
    """dW partial of one shard with the shard offsets applied (what nvfp4_linear_backward_ms_eden does)."""
    tokens = x.shape[0]
    tk = oracle.padded_k(tokens)
    xq = oracle.four_six(x, oracle.row_amax(x), rowwise=True)
    e_t = oracle.ms_eden(1, dy, out_dim, tk, gs_e, SIGN, SCALE ^ 0x85EBCA6B, col_offset=first_token,
                         want_chunk_amax=False)
    gs_x = oracle.ms_eden_global_scale(float(oracle.nvfp4_amax(*xq, tokens, in_dim, True)[1][0]))
    x_t = oracle.ms_eden(3, (*xq, tokens, in_dim), in_dim, tk, gs_x, SIGN, SCALE ^ 0xC2B2AE35, col_offset=first_token,
                         want_chunk_amax=False)
    dw = oracle.gemm(e_t[:3], (x_t[0], x_t[1], np.array([gs_x], np.float32)), out_dim, tk, in_dim, mode=2)
    return dw, e_t


def _worker_sharded(rank, world, port, results):
    oracle, sharding = _setup(rank, world, port)
    x, dy = _data()
    tokens, first = sharding.shard_tokens(TOKENS, world, rank)
    xs, dys = x[first:first + tokens], dy[first:first + tokens]
    # shared global scale of dY: all-reduce(max) of the shard amaxes
    amax = torch.from_numpy(oracle.tensor_amax(dys)[1].copy())
    sharding.sync_amax(amax)
    assert float(amax[0]) == float(np.abs(dy).max())
    gs_e = oracle.ms_eden_global_scale(float(amax[0]))
    # row operand of dY: bit-identical to the slice of the unsharded tensor thanks to the group offset
    ok = oracle.padded_k(OUT_DIM)
    whole = oracle.ms_eden(0, dy, TOKENS, ok, gs_e, SIGN, SCALE, want_chunk_amax=False)
    mine = oracle.ms_eden(0, dys, tokens, ok, gs_e, SIGN, SCALE, want_chunk_amax=False,
                          group_offset=sharding.dy_rows_group_offset(first, OUT_DIM))
    assert np.array_equal(mine[0], whole[0].reshape(TOKENS, -1)[first:first + tokens].reshape(-1))
    assert np.array_equal(mine[1], whole[1].reshape(TOKENS, -1)[first:first + tokens].reshape(-1))
    # dW partial into a gradient bucket, one all-reduce(sum) for the layer
    buckets = sharding.GradBuckets([[(OUT_DIM, IN_DIM, True)]], "cpu")
    dw, e_t = _shard_dw(oracle, xs, dys, gs_e, sharding.dy_transposed_col_offset(first), OUT_DIM, IN_DIM)
    whole_t = oracle.ms_eden(1, dy, OUT_DIM, oracle.padded_k(TOKENS), gs_e, SIGN, SCALE ^ 0x85EBCA6B,
                             want_chunk_amax=False)
    # transposed operand: the shard's nibbles are the matching K slice of the unsharded operand
    assert np.array_equal(e_t[0].reshape(OUT_DIM, -1), whole_t[0].reshape(OUT_DIM, -1)[:, first // 2:(first + tokens) // 2])
    dw_view, db_view = buckets.views[0][0]
    dw_view.copy_(torch.from_numpy(dw))
    db_view.copy_(torch.from_numpy(oracle.bias_grad(dys)))
    buckets.reduce_async(0)
    buckets.wait()
    true_dw, true_db = dy.T @ x, dy.sum(0)
    rel = np.linalg.norm(dw_view.numpy() - true_dw) / np.linalg.norm(true_dw)
    assert rel < 0.3, rel
    assert np.allclose(db_view.numpy(), true_db, rtol=1e-5, atol=1e-7)
    # every rank holds the same reduced bucket
    gathered = [torch.empty_like(buckets.buffers[0]) for _ in range(world)]
    dist.all_gather(gathered, buckets.buffers[0])
    assert all(torch.equal(gathered[0], g) for g in gathered)
    results[rank] = rel
    dist.destroy_process_group()


def _worker_failure(rank, world, port, results):
    _, sharding = _setup(rank, world, port, timeout_s=5)
    buckets = sharding.GradBuckets([[(8, 8, False)]], "cpu")
    if rank == 1:
        results[rank] = "left"
        os._exit(0)  # a rank that leaves between steps, with nothing in flight
    try:
        buckets.reduce_async(0)
        buckets.wait()
        results[rank] = "no error"
    except Exception as exc:  # the survivor learns of it on the host: the collective errors out
        results[rank] = f"error: {type(exc).__name__}"


def _run(worker, world=2):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        if p.is_alive():
            p.terminate()
            pytest.fail("rank did not finish")
    return dict(results), [p.exitcode for p in procs]


def test_shard_plan():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry

    entry.load_package()
    from nanogpt_120a_b200 import sharding

    assert sharding.shard_tokens(65536, 8, 3) == (8192, 24576)
    assert sharding.dy_rows_group_offset(256, 100) == 256 * 8  # K padded to 128 -> 8 groups per row
    with pytest.raises(ValueError):
        sharding.shard_tokens(1000, 2, 0)  # not whole 128-row tiles
    with pytest.raises(ValueError):
        sharding.shard_tokens(1024, 2, 2)


def test_two_rank_sharded_backward_over_gloo():
    results, codes = _run(_worker_sharded)
    assert codes == [0, 0], (results, codes)
    assert set(results) == {0, 1}


def test_rank_failure_is_detected_on_the_host():
    results, _ = _run(_worker_failure)
    assert results.get(1) == "left"
    assert str(results.get(0, "")).startswith("error"), results
