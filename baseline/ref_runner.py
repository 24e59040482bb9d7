"""Runs an unmodified entry script of the reference (the copy under baseline/_ref) for a fixed number of optimizer
steps on synthetic data and times it from the outside.

Nothing of slowrun_b200's models, kernels or engine is on this path. What the harness supplies, without touching
the reference's files, is only what the scripts need to start offline on a B200:
  * a `tiktoken` stand-in (the real one downloads the GPT-2 vocabulary): n_vocab 50257, eot id 50256, fixed byte
    lengths; it only feeds the BPB table;
  * a `wandb` stand-in (the scripts call wandb.init unconditionally on rank 0);
  * a `kernels` stand-in whose `get_kernel` returns an object with `flash_attn_func(q, k, v, causal, window_size
    [, softmax_scale])` backed by the flash-attn 2 wheel of this image, or by torch SDPA if that cannot run here.
    The limited and two-hour scripts only look for FlashAttention-3 when the device reports compute capability 9.x
    and refuse to run otherwise, so the capability query answers (9, 0) until that one lookup is done and is restored
    inside it;
  * for the tiny track, whose loss kernel is compiled at import for compute capability 9.0 only
    (tiny/cuda_kernels.py:305-312): the one `torch.cuda._compile_kernel` call is given this GPU's capability instead,
    from here; the kernel source and the file are untouched;
  * a synthetic Zipf corpus in the reference's .pt format, passed through --input_bin / --input_val_bin.
Timing uses torch's global optimizer-step hooks: a CUDA event and a host timestamp after every `optimizer.step()`;
the period between consecutive steps is one full training step of the script (its micro-batches, H2D copies,
optimizer, loss read-back and logging). After warm-up + timed steps the hook raises to leave the script's loop.
"""
from __future__ import annotations

import json
import os
import runpy
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

SCRIPTS = {"limited": "train.py", "two_hour": os.path.join("two_hour", "train.py"), "tiny": os.path.join("tiny", "train.py")}


class _StopBench(BaseException):
    pass


def reference_available():
    return os.path.isfile(os.path.join(REF_ROOT, "train.py"))


def _install_stubs(state):
    import torch

    tk = types.ModuleType("tiktoken")

    class _Enc:
        n_vocab = 50257
        _special_tokens = {"<|endoftext|>": 50256}

        def decode_single_token_bytes(self, i):
            return b"x" * (1 + (i % 7))

        def encode_ordinary(self, s):
            return [ord(ch) % 50256 for ch in s]

    tk.get_encoding = lambda name: _Enc()
    sys.modules["tiktoken"] = tk

    wb = types.ModuleType("wandb")

    class _Run:
        def __init__(self):
            self.summary = {}
            self.url = None

        def log(self, *a, **k):
            if a and isinstance(a[0], dict):       # kept so that a parity run can read the script's own loss curve
                state.setdefault("wandb_log", []).append(dict(a[0]))

        def log_code(self, *a, **k):
            pass

        def finish(self):
            pass

    wb.init = lambda **kw: _Run()
    sys.modules["wandb"] = wb

    def _sdpa_backend(q, k, v, causal=True, window_size=(-1, -1), softmax_scale=None):
        import torch.nn.functional as F
        T = q.size(1)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        w = window_size[0]
        if w < 0 or w >= T:
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=softmax_scale)
        else:
            i = torch.arange(T, device=q.device).unsqueeze(1)
            j = torch.arange(T, device=q.device).unsqueeze(0)
            y = F.scaled_dot_product_attention(q, k, v, attn_mask=(j <= i) & ((i - j) <= w), scale=softmax_scale)
        return y.transpose(1, 2)

    def _pick_backend():
        if os.environ.get("REF_ATTN", "auto") != "sdpa":
            try:
                from flash_attn import flash_attn_func as fa2
                q = torch.randn(1, 128, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
                y = fa2(q, q, q, causal=True, window_size=(64, 0))
                y.sum().backward()
                torch.cuda.synchronize()
                state["attn_backend"] = "flash_attn2"

                def f(q, k, v, causal=False, window_size=(-1, -1), softmax_scale=None):
                    return fa2(q, k, v, causal=causal, window_size=window_size, softmax_scale=softmax_scale)
                return f
            except Exception as e:  # noqa: BLE001
                state["attn_backend_note"] = f"flash_attn2 unusable: {type(e).__name__}"
        state["attn_backend"] = "torch_sdpa"
        return _sdpa_backend

    real_cap = torch.cuda.get_device_capability
    kn = types.ModuleType("kernels")

    def get_kernel(name, **kw):
        torch.cuda.get_device_capability = real_cap
        return types.SimpleNamespace(flash_attn_func=_pick_backend())

    kn.get_kernel = get_kernel
    sys.modules["kernels"] = kn
    torch.cuda.get_device_capability = lambda *a, **k: (9, 0)
    real_compile = getattr(torch.cuda, "_compile_kernel", None)
    if real_compile is not None:
        def compile_for_this_gpu(*a, **kw):
            kw["compute_capability"] = "".join(str(v) for v in real_cap())
            return real_compile(*a, **kw)
        torch.cuda._compile_kernel = compile_for_this_gpu

    def restore():
        torch.cuda.get_device_capability = real_cap
        if real_compile is not None:
            torch.cuda._compile_kernel = real_compile
    state["restore_cap"] = restore


def run(track: str, steps: int, warmup: int, extra_args, data_dir: str, work_dir: str):
    """Executes the reference script; returns a dict with per-step device/host times (max over ranks) or raises."""
    import torch
    import torch.distributed as dist
    from torch.optim.optimizer import register_optimizer_step_post_hook

    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    if "RANK" not in os.environ:   # the reference's optimizer needs a process group even on one GPU
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(29500 + os.getpid() % 2000))
    state = {}
    _install_stubs(state)
    events, stamps = [], []
    total = warmup + steps

    def post_hook(opt, args, kwargs):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        events.append(ev)
        if len(events) >= warmup:      # host stamps only where they are used; a sync here mirrors the script's own
            torch.cuda.synchronize()
            stamps.append(time.perf_counter())
        if len(events) >= total:
            raise _StopBench()

    handle = register_optimizer_step_post_hook(post_hook)
    script = os.path.join(REF_ROOT, SCRIPTS[track])
    argv = [script, "--input_bin", os.path.join(data_dir, "fineweb_train.pt"),
            "--input_val_bin", os.path.join(data_dir, "fineweb_val.pt")] + list(extra_args)
    old_argv, old_cwd = sys.argv, os.getcwd()
    sys.argv = argv
    sys.path.insert(0, os.path.dirname(script))       # the tiny script imports its kernel module from its own folder
    os.makedirs(work_dir, exist_ok=True)
    os.chdir(work_dir)
    try:
        runpy.run_path(script, run_name="__main__")
        raise RuntimeError("reference script ended before the requested number of steps")
    except _StopBench:
        pass
    finally:
        handle.remove()
        sys.argv = old_argv
        sys.path.remove(os.path.dirname(script))
        os.chdir(old_cwd)
        state["restore_cap"]()
    sys.stdout, sys.stderr = sys.__stdout__, sys.__stderr__
    torch.cuda.synchronize()
    # events[i] is recorded after optimizer.step() of training step i+1; the period events[i-1] -> events[i] is one
    # full step of the script. The timed periods are the `steps` ones after the warm-up steps.
    dev_ms = sum(events[i - 1].elapsed_time(events[i]) for i in range(warmup, total))
    host_s = stamps[-1] - stamps[0]
    t = torch.tensor([dev_ms, host_s * 1000.0], dtype=torch.float64, device="cuda")
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"device_ms": float(t[0]), "host_ms": float(t[1]), "attn_backend": state.get("attn_backend"),
           "note": state.get("attn_backend_note"), "wandb_log": state.get("wandb_log", [])}
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return out
