"""GPTQ row kernel against the float32 restatement of the same algorithm."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(rows, cols, seed):
    torch.manual_seed(seed)
    X = torch.randn(4 * cols, cols, device="cuda") * torch.linspace(0.3, 2.0, cols, device="cuda")
    X = X + 0.5 * X.roll(1, dims=1)                                   # correlated inputs: off-diagonal Hessian mass
    H = X.t() @ X / X.shape[0]
    W = torch.randn(rows, cols, device="cuda") * 0.05
    W[:, 3] *= 6.0                                                    # a few heavy columns so that clipping matters
    return W, H


@pytest.mark.parametrize("rows,cols,bits", [(64, 512, 6), (37, 384, 6), (16, 1536, 5), (8, 200, 6)])
def test_gptq_rows_matches_reference(rows, cols, bits):
    from parameter_golf_b200.ops import native as n
    from parameter_golf_b200.quant.gptq import gptq_prepare, gptq_rows_torch
    W, H = _problem(rows, cols, rows + cols)
    perm, inv_perm, U = gptq_prepare(H)
    Wp = W[:, perm].contiguous()
    qmax = (1 << (bits - 1)) - 1
    scale = (Wp.abs().amax(1) / qmax).clamp_min(1e-8)
    want = gptq_rows_torch(Wp, U, scale, bits)
    got = n.gptq_rows(Wp, U, scale, bits)
    torch.cuda.synchronize()
    assert got.dtype == torch.int8 and got.shape == want.shape
    assert int(got.min()) >= -(qmax + 1) and int(got.max()) <= qmax
    diff = (got.int() - want.int()).abs()
    assert diff.max() <= 1                                              # only rounding-boundary flips from summation order
    assert (diff > 0).float().mean() < 0.01

    def loss(Q):                                                        # the objective GPTQ minimises: tr(E H E^T)
        E = (Wp - Q.float() * scale[:, None]).double()
        Hp = H[perm][:, perm].double()
        return torch.einsum("rc,cd,rd->", E, Hp, E).item()

    assert abs(loss(got) - loss(want)) <= 0.01 * loss(want)
    rtn = (Wp / scale[:, None]).round().clamp(-(qmax + 1), qmax)
    assert loss(got) < loss(rtn)                                        # error feedback beats round-to-nearest


def test_gptq_quantize_uses_the_kernel_on_cuda_tensors():
    from parameter_golf_b200.ops import native as n
    from parameter_golf_b200.quant.gptq import gptq_quantize, gptq_rows_torch
    W, H = _problem(48, 512, 5)
    before = n.launch_count()
    q, s = gptq_quantize(W, H, bits=6)
    assert n.launch_count() - before == 5                               # one launch per clip candidate
    q_ref, s_ref = gptq_quantize(W, H, bits=6, rows_fn=gptq_rows_torch)
    assert torch.allclose(s, s_ref)
    assert ((q.int() - q_ref.int()).abs() > 0).float().mean() < 0.01
