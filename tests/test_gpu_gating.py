"""Gate + sum of the three branches: the CUDA kernels against the reference's eager expression
(oracle.gate_combine restates causal_wan_nsa_model.py:378-386, 541-546)."""
import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(B, M, H, D, dtype, seed, big_logits=True):
    g = torch.Generator().manual_seed(seed)
    gl = torch.randn(B, M, H, 3, generator=g) * (6.0 if big_logits else 1.0)     # some logits beyond +-10
    outs = [torch.randn(B, M, H, D, generator=g) for _ in range(3)]
    return gl.to(dtype), [o.to(dtype) for o in outs]


@pytest.mark.parametrize("mode", ["sigmoid", "softmax"])
@pytest.mark.parametrize("skip", [None, "cmp", "slc"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_matches_the_eager_expression_bit_for_bit(mode, skip, dtype):
    from omnimem_b200.nsa.ops import gated_branch_sum
    gl, (a, b, c) = _inputs(2, 37, 3, 128, dtype, 1)
    want = O.gate_combine(gl, None if skip == "cmp" else a, None if skip == "slc" else b, c, mode)
    dev = torch.device("cuda")
    got = gated_branch_sum(gl.to(dev), a.to(dev), b.to(dev), c.to(dev), mode, skip).cpu()
    # every product and partial sum is rounded like the eager bf16 / fp16 ops: identical up to
    # the last-bit difference of exp() between the CPU and the GPU math libraries
    diff = (got.float() - want.float()).abs()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert (diff <= ulp * want.float().abs().clamp_min(1.0) * 2).all()
    assert (got == want).float().mean() > 0.97


@pytest.mark.parametrize("mode", ["sigmoid", "softmax"])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_backward_matches_autograd_of_the_expression(mode, D):
    from omnimem_b200.nsa.ops import gated_branch_sum
    dtype = torch.bfloat16
    gl, outs = _inputs(1, 64, 4, D, dtype, 2)
    dx = torch.randn(1, 64, 4, D, generator=torch.Generator().manual_seed(3)).to(dtype)
    # reference gradients in fp32 from the same bf16 inputs
    ref_in = [t.float().requires_grad_(True) for t in (gl, *outs)]
    O.gate_combine(ref_in[0], ref_in[1], ref_in[2], ref_in[3], mode).backward(dx.float())
    dev = torch.device("cuda")
    dev_in = [t.to(dev).requires_grad_(True) for t in (gl, *outs)]
    gated_branch_sum(dev_in[0], dev_in[1], dev_in[2], dev_in[3], mode).backward(dx.to(dev))
    for name, r, d in zip(("dg", "do_cmp", "do_slc", "do_swa"), ref_in, dev_in):
        got, want = d.grad.float().cpu(), r.grad
        tol = 2.0 ** -6 * want.abs().max().item() + 1e-3
        assert (got - want).abs().max().item() <= tol, name
    # clamp: no gradient for logits outside [-10, 10]
    outside = (gl.float().abs() > 10)
    assert outside.any()
    assert (dev_in[0].grad.cpu()[outside] == 0).all()


def test_config2_shape_and_errors():
    from omnimem_b200 import ops
    dev = torch.device("cuda")
    gl, (a, b, c) = _inputs(1, 4680, 12, 128, torch.bfloat16, 4, big_logits=False)
    x = ops.gate_combine(gl.to(dev), a.to(dev), b.to(dev), c.to(dev))
    want = O.gate_combine(gl, a, b, c)
    assert (x.cpu() == want).float().mean() > 0.97
    with pytest.raises(NotImplementedError):
        ops.gate_combine(gl.to(dev), a.to(dev), b.to(dev), c.to(dev), "tanh")
    with pytest.raises(ValueError):
        ops.gate_combine(gl.to(dev)[..., :2], a.to(dev), b.to(dev), c.to(dev))
    with pytest.raises(RuntimeError):
        ops.gate_combine(gl.to(dev).float(), a.to(dev).float(), b.to(dev).float(), c.to(dev).float())
