"""Research variants: universal transformer (shared modules, depth schedule) and the gated-delta-rule layer."""
import torch

from slowrun_b200.models.research import (GatedDeltaNetAttention, UniversalConfig, UniversalGPT, depth_at_step,
                                           gated_delta_rule, parse_depth_schedule)


def test_depth_schedule_parsing_and_growth():
    sch = parse_depth_schedule("0:4,10:8")
    assert depth_at_step(sch, 0) == 4 and depth_at_step(sch, 9) == 4 and depth_at_step(sch, 10) == 8
    m = UniversalGPT(UniversalConfig(sequence_len=32, n_layer=8, n_head=2, n_embd=64, depth_schedule="0:4,10:8"))
    assert m.active_n_layer == 4 and m.active_decoder_start == 6
    assert m.apply_depth_schedule(10) and m.active_n_layer == 8 and not m.apply_depth_schedule(11)


def test_universal_gpt_shares_weights_and_trains():
    torch.manual_seed(0)
    m = UniversalGPT(UniversalConfig(sequence_len=32, n_layer=4, n_head=2, n_embd=64, stoch_depth=0.0, depth_schedule="0:4"))
    n_shared = sum(p.numel() for p in list(m.encoder_attns.parameters()) + list(m.encoder_mlp.parameters()))
    n_layer_own = sum(p.numel() for p in m.transformer.h.parameters())
    assert n_shared > 10 * n_layer_own      # the bulk of the parameters is shared across depth
    idx = torch.randint(0, 50257, (2, 32))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    first = None
    for _ in range(8):
        loss = m(idx, idx)
        first = first if first is not None else loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < first
    assert m.encoder_attns[0].c_q.weight.grad.abs().sum() > 0


def test_gated_delta_rule_matches_explicit_recurrence_and_is_causal():
    torch.manual_seed(0)
    B, T, H, D = 1, 6, 2, 4
    q, k, v = torch.randn(B, T, H, D), torch.nn.functional.normalize(torch.randn(B, T, H, D), dim=-1), torch.randn(B, T, H, D)
    alpha, beta = torch.rand(B, T, H) * 0.5 + 0.5, torch.rand(B, T, H)
    o = gated_delta_rule(q, k, v, alpha, beta)
    S = torch.zeros(H, D, D)
    for t in range(T):
        for h in range(H):
            kk = k[0, t, h]
            S[h] = alpha[0, t, h] * S[h] @ (torch.eye(D) - beta[0, t, h] * torch.outer(kk, kk)) + beta[0, t, h] * torch.outer(v[0, t, h], kk)
            assert torch.allclose(o[0, t, h], S[h] @ q[0, t, h], atol=1e-5)
    layer = GatedDeltaNetAttention(32, 2)
    x = torch.randn(1, 8, 32)
    y1 = layer(x)
    x2 = x.clone()
    x2[:, 5:] += 1.0
    assert torch.allclose(layer(x2)[:, :5], y1[:, :5], atol=1e-5)   # later tokens cannot influence earlier outputs
