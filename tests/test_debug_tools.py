"""The memory-checker and race-detector stand-ins (slowrun_b200/utils/debug.py) on the CPU path: red zones around every
buffer the op layer allocates stay intact through a training step, a store past a buffer's end is caught and attributed,
and repeated runs of the same step are bit-identical."""
import pytest
import torch

from slowrun_b200.config import track_defaults
from slowrun_b200.models.gpt import build_model
from slowrun_b200.utils.debug import RedZones, repeat_check


def _model(track="limited"):
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 2, 64, 2, 2, 48
    m.dropout, m.stoch_depth = 0.0, 0.0
    return build_model(m, torch.device("cpu"), seed=0)


def test_red_zones_survive_a_training_step_and_catch_an_overrun():
    model = _model()
    idx = torch.randint(0, 50257, (2, 49))
    with RedZones() as zones:
        loss, _ = model(idx[:, :-1], idx[:, 1:])
        loss.backward()
        buf = torch.empty(37, dtype=torch.bfloat16)
        assert zones.check() >= 1
        # a store one element past the end, made through the enclosing byte buffer (legal memory: the guard itself)
        raw, g, nbytes, _ = zones.records[-1]
        assert nbytes == 74 and buf.data_ptr() == raw.data_ptr() + g
        raw[g + nbytes + (-nbytes) % 16] = 0
        with pytest.raises(AssertionError, match="after the 74-byte buffer allocated at test_debug_tools.py"):
            zones.check()
    assert torch.empty is not None and torch.empty(3).shape == (3,)       # the allocation functions are restored


def test_repeat_check_passes_for_a_deterministic_step_and_flags_a_varying_one():
    model = _model()
    idx = torch.randint(0, 50257, (2, 49))

    def step():
        model.zero_grad(set_to_none=True)
        loss, _ = model(idx[:, :-1], idx[:, 1:])
        loss.backward()
        return [loss.detach()] + [p.grad for p in model.parameters() if p.grad is not None]

    repeat_check(step, times=3)
    calls = []

    def noisy():
        calls.append(1)
        return torch.full((4,), float(len(calls)))

    with pytest.raises(AssertionError, match="run 1 differs from run 0"):
        repeat_check(noisy, times=2)
    repeat_check(noisy, times=2, atol=10.0)
