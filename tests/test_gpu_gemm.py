"""tcgen05 GEMM against an fp32 PyTorch reference: operand majors, batch, split-K, every epilogue, ragged edges."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _n():
    from parameter_golf_b200.ops import native
    return native


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _ref(A, B, a_k, b_k):
    Af = A.float() if a_k else A.float().transpose(-1, -2)
    Bf = B.float() if b_k else B.float().transpose(-1, -2)
    return Af @ Bf.transpose(-1, -2)


def _close(got, ref, rel=1e-2):
    err = (got.float() - ref).abs().max().item()
    assert err <= rel * max(ref.abs().max().item(), 1e-3), f"max abs err {err} vs ref max {ref.abs().max().item()}"


@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 512, 192), (200, 136, 72), (128, 1024, 512), (1000, 64, 64)])
def test_gemm_majors_and_ragged_shapes(a_k, b_k, M, N, K):
    n = _n()
    torch.manual_seed(M + N + K)
    A = _rand(M, K) if a_k else _rand(K, M)
    B = _rand(N, K) if b_k else _rand(K, N)
    D = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    n.gemm(A, B, D, a_k, b_k)
    torch.cuda.synchronize()
    n.check_status()
    _close(D, _ref(A, B, a_k, b_k))


def test_gemm_batched_strided_and_fp32_out():
    n = _n()
    A, B = _rand(5, 256, 320), _rand(5, 384, 320)
    D = torch.empty(5, 256, 384, device="cuda", dtype=torch.float32)
    n.gemm(A, B, D, True, True, n.EPI_F32, alpha=0.5)
    torch.cuda.synchronize()
    n.check_status()
    _close(D, 0.5 * _ref(A, B, True, True), 3e-3)
    big = _rand(4, 256, 640)                      # batch stride larger than rows*cols, row stride larger than K
    Av = big[:, :, :320]
    D2 = torch.empty(4, 256, 384, device="cuda", dtype=torch.bfloat16)
    n.gemm(Av, B[:4], D2, True, True)
    torch.cuda.synchronize()
    _close(D2, _ref(Av, B[:4], True, True))


@pytest.mark.parametrize("splits", [0, 1, 3, 8])
def test_split_k_weight_gradient_accumulates(splits):
    """dW[N,K] += dY^T X: both operands row-contiguous along the output dims, reduction over tokens."""
    n = _n()
    T, N, K = 4096, 256, 192
    dY, X = _rand(T, N, scale=0.1), _rand(T, K)
    dW = torch.ones(N, K, device="cuda", dtype=torch.float32)
    n.gemm(dY, X, dW, False, False, n.EPI_F32_ATOMIC, splits=splits)
    n.gemm(dY, X, dW, False, False, n.EPI_F32_ATOMIC, splits=splits)
    torch.cuda.synchronize()
    n.check_status()
    _close(dW, 1.0 + 2.0 * (dY.float().t() @ X.float()), 3e-3)


def test_epilogue_axpby_residual_activation():
    n = _n()
    M, N, K = 384, 512, 256
    A, B, aux = _rand(M, K), _rand(N, K, scale=0.1), _rand(M, N)
    ref = _ref(A, B, True, True)
    D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    n.gemm(A, B, D, epi=n.EPI_AXPBY_BF16, alpha=0.7, beta=-1.3, aux=aux)
    _close(D, 0.7 * ref - 1.3 * aux.float())
    cs = torch.randn(N, device="cuda")
    n.gemm(A, B, D, epi=n.EPI_RESID_BF16, aux=aux, colscale=cs)
    _close(D, aux.float() + cs[None, :] * ref)
    H, Act = torch.empty_like(D), torch.empty_like(D)
    n.gemm(A, B, H, epi=n.EPI_ACT_SQ, slope=0.5, D2=Act)
    _close(H, ref)
    _close(Act, torch.nn.functional.leaky_relu(H.float(), 0.5) ** 2, 1e-2)
    G = torch.empty_like(D)
    n.gemm(A, B, G, epi=n.EPI_MUL_ACTGRAD, slope=0.5, aux=aux)
    h = aux.float()
    _close(G, ref * 2 * torch.nn.functional.leaky_relu(h, 0.5) * torch.where(h >= 0, 1.0, 0.5))
    n.gemm(A, B, Act, epi=n.EPI_ACT_SQ, slope=0.0, D2=G)           # relu^2
    _close(G, torch.relu(Act.float()) ** 2)
    torch.cuda.synchronize()
    n.check_status()


def test_many_tiles_persistent_schedule_matches():
    """More tiles than SMs so every CTA loops over several tiles and both accumulators are used."""
    n = _n()
    M, N, K = 128 * 40, 1024, 512
    A, B = _rand(M, K), _rand(N, K, scale=0.05)
    D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    n.gemm(A, B, D)
    torch.cuda.synchronize()
    n.check_status()
    _close(D, _ref(A, B, True, True))


def test_row_segments_scatter_one_product_into_three_gradient_matrices():
    """dW of a packed [q; k; v] projection: rows 0..255 / 256..383 / 384..511 of the product accumulate into three matrices."""
    n = _n()
    torch.manual_seed(3)
    T, d, dq, dkv = 4096, 192, 256, 128
    dY, X = _rand(T, dq + 2 * dkv, scale=0.3), _rand(T, d, scale=0.3)
    bank = torch.randn(dq + 2 * dkv + 64, d, device="cuda")                  # three slots of one fp32 buffer, out of order
    Gq, Gk, Gv = bank[dkv + 64:dkv + 64 + dq], bank[:dkv], bank[dkv + 64 + dq:]
    before = bank.clone()
    n.gemm(dY, X, Gq, False, False, n.EPI_F32_ATOMIC, segs=((dq, Gk), (dq + dkv, Gv)))
    torch.cuda.synchronize()
    n.check_status()
    ref = dY.float().t() @ X.float()
    upd = bank - before
    _close(upd[dkv + 64:dkv + 64 + dq], ref[:dq], 5e-3)
    _close(upd[:dkv], ref[dq:dq + dkv], 5e-3)
    _close(upd[dkv + 64 + dq:], ref[dq + dkv:], 5e-3)
    assert upd[dkv:dkv + 64].abs().max().item() == 0.0                        # the gap between the slots is untouched


def test_gemm_producer_gives_up_on_a_weight_flag_nobody_sets_and_the_context_survives():
    """The weight operand of a QKV product may be gated on a ready counter that peer ranks bump. If it never reaches the
    expected value the producer warp's bounded wait runs out: the kernel reports to the status word, every role unwinds
    (no tensor-memory or bulk-copy state is left behind) and the next product on the same context is correct."""
    from parameter_golf_b200.ops import native as n
    torch.manual_seed(0)
    A = (torch.randn(512, 512, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(1024, 512, device="cuda") * 0.5).bfloat16()
    D = torch.zeros(512, 1024, device="cuda", dtype=torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    n.status_word().zero_()
    n.gemm(A, W, D, wait_flag=flag, wait_value=3)            # nothing ever bumps the flag
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="wait_flag"):
        n.check_status()
    flag.fill_(3)
    n.gemm(A, W, D, wait_flag=flag, wait_value=3)
    torch.cuda.synchronize()
    n.check_status()
    ref = A.float() @ W.float().t()
    assert (D.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item()


@pytest.mark.parametrize("T,d,H,Hkv,rope,S", [(1000, 512, 8, 4, 16, 250), (384, 128, 2, 1, 16, 128), (257, 192, 1, 1, 0, 257), (640, 256, 4, 4, 64, 128),
                                              (300, 128, 2, 2, 32, 100)])
def test_qkv_product_with_norm_rope_and_gain_in_its_output_stage(T, d, H, Hkv, rope, S):
    """pre = h W^T and post = gain * rope(rms_norm(pre)) from one kernel, against the plain product followed by the row kernel,
    and against the fp32 reference of the op."""
    from parameter_golf_b200.ops import reference as R
    n = _n()
    C = n.load()
    hd, eps = 64, 1e-6
    N = (H + 2 * Hkv) * hd
    h, W = _rand(T, d), _rand(N, d, scale=d ** -0.5)
    gain = torch.rand(H, device="cuda") + 0.75
    cos = sin = None
    if rope:
        cos, sin = R.rope_tables(S, rope, 10000.0, device="cuda")
        cos, sin = cos.contiguous(), sin.contiguous()
    pre, post = torch.full((T, N), 7.0, device="cuda", dtype=torch.bfloat16), torch.full((T, N), 7.0, device="cuda", dtype=torch.bfloat16)
    n.gemm_qkv_norm_rope(h, W, pre, post, cos, sin, gain, H, Hkv, rope, S, eps)
    pre2, post2 = torch.empty_like(pre), torch.full_like(post, 7.0)
    n.gemm(h, W, pre2)
    C.qk_norm_rope_fwd(pre2, post2, cos, sin, gain, H, Hkv, hd, rope, S, eps)
    torch.cuda.synchronize()
    n.check_status()
    assert torch.equal(pre, pre2)
    qk = (H + Hkv) * hd
    assert torch.equal(post[:, qk:], torch.full_like(post[:, qk:], 7.0))            # the value columns of post are not touched
    assert (post[:, :qk].float() - post2[:, :qk].float()).abs().max() < 0.02
    if T % S == 0:
        B = T // S
        qf = pre[:, :H * hd].float().reshape(B, S, H, hd)
        kf = pre[:, H * hd:qk].float().reshape(B, S, Hkv, hd)
        q_ref, k_ref = R.qk_norm_rope_gain(qf, kf, cos, sin, rope, gain, eps)
        _close(post[:, :H * hd], q_ref.reshape(T, H * hd))
        _close(post[:, H * hd:qk], k_ref.reshape(T, Hkv * hd))
