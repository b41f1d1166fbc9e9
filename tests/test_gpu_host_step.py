"""The C++ training-step driver (include/nvfp4_b200_step.hpp, no PyTorch on its path) against the Python
`ProjectionSet` that issues the same C-ABI calls one by one: same inputs, same seed stream, identical gradient
buckets and dX tensors, byte for byte, over two consecutive steps (the seeds advance)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(pkg, dev, fused_mlp, tokens=256, **kw):
    from nanogpt_120a_b200.host_step import HostStep
    from nanogpt_120a_b200.projection_set import ModelShape, ProjectionSet

    shape = ModelShape("tiny-proj-set", 2, 128, 256, 512)
    a = ProjectionSet(shape, tokens, dev, seed=5, fused_mlp=fused_mlp, **kw)
    b = ProjectionSet(shape, tokens, dev, seed=5, fused_mlp=fused_mlp, **kw)
    return a, b, HostStep(b)


@pytest.mark.parametrize("fused_mlp", [True, False])
def test_cpp_step_equals_python_step(pkg, dev, fused_mlp):
    a, b, host = _pair(pkg, dev, fused_mlp)
    for step in range(2):
        a.step()
        host.step()
        torch.cuda.synchronize()
        for x, y in zip(a.buckets, host.buckets):
            assert torch.equal(x, y), step
        for w in a.dx:
            assert torch.equal(a.dx[w], host.dx(w)), (step, w)
    assert host.flops_per_step() == a.flops_per_step()
    assert pkg.read_device_status() == 0
    host.close()


def test_cpp_step_keeps_packed_weights_and_swaps_inputs(pkg, dev):
    """weights_changed = 0 reuses the packed weights (same gradients, fewer launches); set_inputs swaps the
    activation / gradient tensors a step reads."""
    a, b, host = _pair(pkg, dev, True)
    a.step()
    host.step()
    n0 = pkg.launch_count()
    host.step(weights_changed=True)
    n1 = pkg.launch_count()
    a.step()
    a.step(weights_changed=False)
    n2 = pkg.launch_count()
    host.step(weights_changed=False)
    n3 = pkg.launch_count()
    torch.cuda.synchronize()
    assert (n1 - n0) - (n3 - n2) >= len(a.all_linears())
    for x, y in zip(a.buckets, host.buckets):
        assert torch.equal(x, y)
    # other inputs: scaled copies; the Python set reads the same tensors
    x2 = {w: (t.float() * 0.5).to(torch.bfloat16) for w, t in a.x.items()}
    dy2 = {w: (t.float() * 2.0).to(torch.bfloat16) for w, t in a.dy.items()}
    a.x, a.dy = x2, dy2
    host.set_inputs(x2, dy2)
    a.step()
    host.step()
    torch.cuda.synchronize()
    for x, y in zip(a.buckets, host.buckets):
        assert torch.equal(x, y)
    host.close()


def test_cpp_step_reproducible_sharding_single_rank(pkg, dev):
    """With one rank the reproducible-sharding path (amax vector, scales from it, unsharded index spaces) must
    give the bits of the plain path: the all-reduce is the identity."""
    a, b, host = _pair(pkg, dev, True)
    c, d, host_r = _pair(pkg, dev, True, total_tokens=256, reproducible_sharding=True)
    a.step()
    c.step()
    host.step()
    host_r.step()
    torch.cuda.synchronize()
    for w, x, y, z in zip(a.buckets, c.buckets, host.buckets, host_r.buckets):
        assert torch.equal(w, x) and torch.equal(w, y) and torch.equal(w, z)
    host.close()
    host_r.close()
