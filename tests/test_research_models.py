"""Research variants: universal transformer (shared modules, depth schedule) and the gated delta rule."""
import torch

from slowrun_b200.models.research import UniversalConfig, UniversalGPT, depth_at_step, parse_depth_schedule
from slowrun_b200.ops.linear_attention import gated_delta_rule_recurrent


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


def test_gated_delta_rule_definition_matches_an_explicit_matrix_recurrence():
    """S_t = diag(a_t) S_{t-1} (then) S_t += b_t k_t (v_t - S_t^T k_t)^T ; o_t = S_t^T q_t, written with plain matrices."""
    torch.manual_seed(0)
    B, T, H, Dk, Dv = 1, 6, 2, 4, 3
    q, k, v = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1), torch.randn(B, T, H, Dv)
    g, beta = -torch.rand(B, T, H), torch.rand(B, T, H) * 2
    o = gated_delta_rule_recurrent(q, k, v, g, beta)
    for h in range(H):
        S = torch.zeros(Dk, Dv)
        for t in range(T):
            S = torch.exp(g[0, t, h]) * S
            S = S + beta[0, t, h] * torch.outer(k[0, t, h], v[0, t, h] - S.t() @ k[0, t, h])
            assert torch.allclose(o[0, t, h], S.t() @ q[0, t, h], atol=1e-5)
