"""GPU numerics of the gated-delta-rule recurrence kernel against the token-by-token fp32 definition, for both decay
forms (one log-decay per head: Gated DeltaNet; one per key channel: Kimi Delta Attention), both key widths the kernel
is built for, and of the op's backward (chunked re-derivation) against autograd through the definition."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, Dk, Dv, per_channel, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    q = (torch.nn.functional.normalize(r(B, T, H, Dk), dim=-1) * Dk ** -0.5).bfloat16()
    k = torch.nn.functional.normalize(r(B, T, H, Dk), dim=-1).bfloat16()
    v = r(B, T, H, Dv).bfloat16()
    decay = -torch.rand(B, T, H, Dk, device="cuda", generator=g) * 2 if per_channel else -torch.rand(B, T, H, device="cuda", generator=g)
    beta = torch.rand(B, T, H, device="cuda", generator=g) * 2
    return q, k, v, decay, beta


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("B,T,H,Dk,Dv", [(2, 70, 3, 64, 128), (1, 257, 2, 128, 128), (1, 33, 2, 64, 20)])
def test_recurrence_kernel_matches_definition(per_channel, B, T, H, Dk, Dv):
    from slowrun_b200.ops import _lib
    from slowrun_b200.ops.linear_attention import gated_delta_rule, gated_delta_rule_recurrent
    q, k, v, g, beta = _inputs(B, T, H, Dk, Dv, per_channel)
    with torch.no_grad():
        o = gated_delta_rule(q, k, v, g, beta)
    ref = gated_delta_rule_recurrent(q.float(), k.float(), v.float(), g, beta)
    torch.cuda.synchronize()
    _lib.check_status()
    rel = ((o.float() - ref).norm() / ref.norm()).item()
    assert rel < 1e-2, rel


def test_op_backward_matches_autograd_through_the_definition():
    from slowrun_b200.ops.linear_attention import gated_delta_rule, gated_delta_rule_recurrent
    q, k, v, g, beta = _inputs(1, 48, 2, 64, 32, False, seed=3)
    ins = [t.float().requires_grad_(True) for t in (q, k, v, g, beta)]
    o = gated_delta_rule(*ins)                       # CUDA kernel forward, chunked backward
    w = torch.randn_like(o)
    grads = torch.autograd.grad((o * w).sum(), ins)
    ins2 = [t.detach().clone().requires_grad_(True) for t in ins]
    o2 = gated_delta_rule_recurrent(*ins2)
    grads2 = torch.autograd.grad((o2 * w).sum(), ins2)
    assert ((o - o2).norm() / o2.norm()).item() < 1e-2        # the kernel takes bf16 operands
    for a, b in zip(grads, grads2):
        assert ((a - b).norm() / b.norm().clamp_min(1e-9)).item() < 2e-3
