"""The delta-rule state-scan kernels (forward and backward) against the same loop on fp32 PyTorch ops, and the chunked scan
built on them against the token-by-token recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiles(B, H, N, dk, dv, seed=0, with_state=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s, scale=1.0: (torch.randn(*s, device="cuda", generator=g) * scale).requires_grad_()  # noqa: E731
    w, qg, kd = r(B, H, N, 64, dk, scale=0.03), r(B, H, N, 64, dk, scale=0.1), r(B, H, N, 64, dk, scale=0.03)
    P = (torch.randn(B, H, N, 64, 64, device="cuda", generator=g) * 0.1).tril().requires_grad_()
    u = r(B, H, N, 64, dv)
    a = (torch.rand(B, H, N, device="cuda", generator=g) * 0.4 + 0.4).requires_grad_()
    S0 = r(B, H, dk, dv, scale=0.5) if with_state else None
    return [w, qg, kd, P, u, a, S0]


def _run(fn, args, go, gs):
    for t in args:
        if t is not None:
            t.grad = None
    out, S = fn(*args)
    (out * go).sum().add((S * gs).sum()).backward()
    return out.detach(), S.detach(), [None if t is None else t.grad.clone() for t in args]


@pytest.mark.parametrize("exact", [True, False])
@pytest.mark.parametrize("B,H,N,dk,dv,with_state", [(1, 2, 3, 128, 128, True), (2, 3, 5, 64, 64, False), (1, 1, 2, 64, 192, True)])
def test_state_scan_kernel_matches_fp32_loop(B, H, N, dk, dv, with_state, exact):
    from levanter_b200.ops import lib
    from levanter_b200.ops.delta_rule import chunk_state_scan, chunk_state_scan_reference

    args = _tiles(B, H, N, dk, dv, with_state=with_state)
    go = torch.randn(B, H, N, 64, dv, device="cuda")
    gs = torch.randn(B, H, dk, dv, device="cuda")
    o_ref, s_ref, g_ref = _run(chunk_state_scan_reference, args, go, gs)
    n0 = lib.launch_count
    o, s, grads = _run(lambda *a: chunk_state_scan(*a, exact=exact), args, go, gs)
    assert lib.launch_count - n0 == 2  # one kernel per direction
    lib.check_status()
    tol = 2e-4 if exact else 1e-2  # TF32 products: 10-bit mantissas on the operands, fp32 accumulation

    def close(x, y, what):
        err = (x - y).abs().max().item()
        scale = y.abs().max().item() + 1e-6
        assert err <= tol * scale, f"{what}: max err {err:.3e} against scale {scale:.3e}"

    close(o, o_ref, "out")
    close(s, s_ref, "final state")
    for name, x, y in zip(["dw", "dqg", "dkd", "dP", "du", "da", "dS0"], grads, g_ref):
        if y is not None:
            if name == "dP":  # entries above the diagonal never reach the caller (the scores are masked there)
                x, y = x.tril(), y.tril()
            close(x, y, name)


def test_state_scan_is_bitwise_reproducible():
    from levanter_b200.ops.delta_rule import chunk_state_scan

    args = _tiles(2, 2, 4, 128, 128, seed=3)
    go = torch.randn(2, 2, 4, 64, 128, device="cuda")
    gs = torch.zeros(2, 2, 128, 128, device="cuda")
    first = _run(chunk_state_scan, args, go, gs)
    second = _run(chunk_state_scan, args, go, gs)
    assert torch.equal(first[0], second[0]) and torch.equal(first[1], second[1])
    for x, y in zip(first[2], second[2]):
        assert torch.equal(x, y)


def test_chunked_scan_on_kernels_matches_recurrence():
    from levanter_b200.models.gated_deltanet import delta_rule_chunked_scan, delta_rule_recurrent

    torch.manual_seed(0)
    B, H, L, dk, dv = 2, 2, 200, 128, 128  # L is not a multiple of the chunk: the tail is padded
    q = torch.nn.functional.normalize(torch.randn(B, H, L, dk, device="cuda"), dim=-1).requires_grad_()
    k = torch.nn.functional.normalize(torch.randn(B, H, L, dk, device="cuda"), dim=-1).requires_grad_()
    v = torch.randn(B, H, L, dv, device="cuda").requires_grad_()
    g = (-torch.rand(B, H, L, device="cuda") * 0.1).requires_grad_()
    beta = torch.rand(B, H, L, device="cuda").requires_grad_()
    go = torch.randn(B, H, L, dv, device="cuda")

    def run(fn):
        for t in (q, k, v, g, beta):
            t.grad = None
        o, S = fn(q, k, v, g, beta)
        (o * go).sum().backward()
        return o.detach(), S.detach(), [t.grad.clone() for t in (q, k, v, g, beta)]

    o_ref, s_ref, g_ref = run(delta_rule_recurrent)
    o, s, grads = run(delta_rule_chunked_scan)
    torch.testing.assert_close(o, o_ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(s, s_ref, atol=2e-2, rtol=2e-2)
    for x, y in zip(grads, g_ref):
        assert (x - y).abs().max().item() <= 2e-2 * (y.abs().max().item() + 1e-6)
