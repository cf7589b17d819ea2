"""The allocation-free C entry point of the attention backward, called through its exported symbol.

Collected last on purpose (file name): it must pass alone and after every other GPU test has used the device.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

HD = 64


def _lib():
    from parameter_golf_b200.ops import native as n
    n.load()                                   # builds / imports the extension and fails loudly when it is missing
    import parameter_golf_b200._C as ext
    lib = ctypes.CDLL(ext.__file__)
    ll, i, vp = ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p
    lib.pgb_attn_bwd_noalloc.argtypes = [vp] * 9 + [ll] * 8 + [i] * 6 + [vp, vp]
    lib.pgb_attn_bwd_noalloc.restype = i
    lib.pgb_attn_bwd_noalloc_setup.restype = i
    lib.pgb_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(B, S, H, Hkv, seed):
    from parameter_golf_b200.ops import native as n
    torch.manual_seed(seed)
    qkv = (torch.randn(B * S, (H + 2 * Hkv) * HD, device="cuda") * 1.2).bfloat16()
    q, k, v = qkv[:, :H * HD], qkv[:, H * HD:(H + Hkv) * HD], qkv[:, (H + Hkv) * HD:]
    o = torch.empty(B * S, H * HD, device="cuda", dtype=torch.bfloat16)
    lse = n.attn_fwd(q, k, v, o, B, S, H, Hkv, HD)
    d_o = torch.randn(B * S, H * HD, device="cuda").bfloat16()
    return q, k, v, o, d_o, lse


def _call(lib, q, k, v, o, d_o, lse, dq, dk, dv, B, S, H, Hkv, accumulate=0):
    from parameter_golf_b200.ops import native as n
    st = n.status_word(q.device)
    return lib.pgb_attn_bwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(), dq.data_ptr(),
                                    dk.data_ptr(), dv.data_ptr(), q.stride(0), k.stride(0), v.stride(0), o.stride(0), d_o.stride(0), dq.stride(0),
                                    dk.stride(0), dv.stride(0), B, S, H, Hkv, HD, accumulate, st.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)


def test_matches_regular_entry_point_twice_in_a_row():
    from parameter_golf_b200.ops import native as n
    lib = _lib()
    assert lib.pgb_attn_bwd_noalloc_setup() == 0, lib.pgb_noalloc_last_error()
    # two different problems back to back: the second call finds the first one's leftovers in the shared scratch
    cases = [(2, 384, 4, 2, 11), (1, 640, 8, 4, 12)]
    prepared = []
    for B, S, H, Hkv, seed in cases:
        q, k, v, o, d_o, lse = _case(B, S, H, Hkv, seed)
        want = [torch.empty(B * S, H * HD, device="cuda", dtype=torch.bfloat16), torch.empty(B * S, Hkv * HD, device="cuda", dtype=torch.bfloat16),
                torch.empty(B * S, Hkv * HD, device="cuda", dtype=torch.bfloat16)]
        n.attn_bwd(q, k, v, o, d_o, lse, *want, B, S, H, Hkv, HD, reproducible=True)
        got = [torch.zeros_like(t) for t in want]
        prepared.append((q, k, v, o, d_o, lse, want, got, B, S, H, Hkv))
    torch.cuda.synchronize()
    n.check_status()
    allocated = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    for q, k, v, o, d_o, lse, want, got, B, S, H, Hkv in prepared:
        rc = _call(lib, q, k, v, o, d_o, lse, *got, B, S, H, Hkv)
        assert rc == 0, lib.pgb_noalloc_last_error()
    torch.cuda.synchronize()
    n.check_status()
    assert torch.cuda.memory_allocated() == allocated
    assert torch.cuda.mem_get_info()[0] == free_before          # nothing was taken from the driver either
    for *_, want, got, B, S, H, Hkv in prepared:
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            assert torch.equal(a, b), (name, (a.float() - b.float()).abs().max().item())


def test_accumulating_into_dv_matches():
    from parameter_golf_b200.ops import native as n
    lib = _lib()
    B, S, H, Hkv = 1, 256, 2, 1
    q, k, v, o, d_o, lse = _case(B, S, H, Hkv, 5)
    base = torch.randn(B * S, Hkv * HD, device="cuda").bfloat16()
    want = [torch.empty(B * S, H * HD, device="cuda", dtype=torch.bfloat16), torch.empty(B * S, Hkv * HD, device="cuda", dtype=torch.bfloat16), base.clone()]
    got = [torch.empty_like(want[0]), torch.empty_like(want[1]), base.clone()]
    n.attn_bwd(q, k, v, o, d_o, lse, *want, B, S, H, Hkv, HD, accumulate_dv=True, reproducible=True)
    assert _call(lib, q, k, v, o, d_o, lse, *got, B, S, H, Hkv, accumulate=1) == 0, lib.pgb_noalloc_last_error()
    torch.cuda.synchronize()
    n.check_status()
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_rejects_problems_beyond_the_scratch_without_launching():
    lib = _lib()
    B, S, H, Hkv = 64, 4096, 8, 4                    # 2 Mi rows > 1 Mi
    dummy = torch.zeros(8, device="cuda")
    p = dummy.data_ptr()
    rc = lib.pgb_attn_bwd_noalloc(p, p, p, p, p, p, p, p, p, 512, 256, 256, 512, 512, 512, 256, 256, B, S, H, Hkv, HD, 0, None, None)
    assert rc == 1
    msg = lib.pgb_noalloc_last_error().decode()
    assert "exceeds" in msg and str(1 << 20) in msg
    assert lib.pgb_attn_bwd_noalloc(p, p, p, p, p, p, p, p, p, 512, 256, 256, 512, 512, 512, 256, 256, 1, 100, 8, 4, HD, 0, None, None) == 2
    torch.cuda.synchronize()
