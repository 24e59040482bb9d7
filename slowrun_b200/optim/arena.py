"""Stacked parameter / gradient / bf16-shadow arenas.

Every Muon shape group lives in three contiguous buffers laid out in the optimizer's member order:
  P   [n, r, c]      fp32 master parameters (each nn.Parameter's .data is a view of its slot)
  G   [n_pad, r, c]  fp32 gradients, padded to a multiple of the world size (each .grad is a view)
  W16 [n, r, c]      bf16 shadows the forward/backward GEMMs read (CUDA only)
so the per-rank chunk of a reduce-scatter, the owned stack of a Muon step and the fused [c_q;c_k;c_v] /
[c_gate;c_fc] GEMM operands are all plain slices: nothing is stacked or copied per step. The reference re-stacks
every gradient and every owned parameter on each step (train.py:677-680, 730, 760).
With more than one rank the members of a group are ordered by (layer mod world, layer): rank r's contiguous chunk then
holds layers r, r + world, ... instead of a block of neighbouring layers, so that while the backward pass walks down
the network every rank's matrices become final at an even pace and their reduction can run under the rest of the
pass (`ShardedMuonAdamW.begin_backward_overlap`). Which rank owns which matrix is internal; results do not depend on it.
Small parameters (numel < 1024: scalars, IHA mixes, gates) share one flat gradient buffer so they need a single
all-reduce (the reference issues one per tensor, train.py:660-662).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .groups import muon_shape_groups

SMALL_NUMEL = 1024


def layer_of_param(model) -> Dict[int, int]:
    """id(parameter) -> index of the layer that writes its gradient (n_layer for the extra prediction block)."""
    owner = {}
    h = model.transformer.h
    for i, blk in enumerate(h):
        for p in blk.parameters():
            owner[id(p)] = i
    for k, lin in getattr(model, "ve_projs", {}).items():
        owner[id(lin.weight)] = int(k)
    if getattr(model, "mtp_weight", 0) > 0 and hasattr(model, "mtp_block"):
        for p in list(model.mtp_block.parameters()) + list(model.mtp_proj.parameters()):
            owner[id(p)] = len(h)
    return owner


class MuonGroupArena:
    def __init__(self, shape, params: List[torch.nn.Parameter], world_size: int, make_shadow: bool, zeros=None,
                 layer_of=None):
        self.shape = tuple(shape)
        if world_size > 1 and layer_of is not None:
            key = {id(p): (layer_of.get(id(p), 0) % world_size, layer_of.get(id(p), 0), i) for i, p in enumerate(params)}
            params = sorted(params, key=lambda p: key[id(p)])
        self.params = params
        self.layers = [layer_of.get(id(p)) if layer_of is not None else None for p in params]
        n = len(params)
        r, c = self.shape
        dev = params[0].device
        self.n = n
        self.chunk = (n + world_size - 1) // world_size
        self.n_pad = self.chunk * world_size
        self.P = torch.empty((n, r, c), dtype=torch.float32, device=dev)
        self.G = (zeros or (lambda sh, dt: torch.zeros(sh, dtype=dt, device=dev)))((self.n_pad, r, c), torch.float32)
        self.W16 = torch.empty((n, r, c), dtype=torch.bfloat16, device=dev) if make_shadow else None
        for i, p in enumerate(params):
            self.P[i].copy_(p.data)
            p.data = self.P[i]
            p.grad = self.G[i]
        if self.W16 is not None:
            self.W16.copy_(self.P)

    def index_of(self, p) -> int:
        for i, q in enumerate(self.params):
            if q is p:
                return i
        raise KeyError("parameter not in group")


class ParamArena:
    def __init__(self, model, world_size: int = 1, alloc=None):
        """`alloc(shape, dtype)` (optional) returns zero-filled peer-mapped memory; everything another rank has to read
        (gradients, the sharded AdamW parameters) is then placed there."""
        self.model = model
        self.world_size = world_size
        dev = model.get_device()
        cuda = dev.type == "cuda"
        self.symmetric = alloc is not None

        def zeros(shape, dtype):
            if alloc is not None:
                return alloc(tuple(shape), dtype)
            return torch.zeros(tuple(shape), dtype=dtype, device=dev)

        def repoint(p):
            if alloc is not None:
                buf = alloc(tuple(p.shape), p.dtype)
                buf.copy_(p.data)
                p.data = buf
        self.groups: Dict[tuple, MuonGroupArena] = {}
        self.alloc = alloc
        layer_of = layer_of_param(model) if hasattr(model, "transformer") else None
        for shape, ps in muon_shape_groups(model):
            big = cuda and shape[0] % 8 == 0 and shape[1] % 8 == 0 and shape[1] >= 64 and shape[0] >= 64
            self.groups[tuple(shape)] = MuonGroupArena(shape, ps, world_size, make_shadow=big, zeros=zeros, layer_of=layer_of)
        # lm head
        head = model.lm_head.weight
        self.head_w16 = None
        repoint(head)
        if head.dtype == torch.float32:
            head.grad = zeros(head.shape, torch.float32)
            self.head_grad = head.grad
            if cuda:
                self.head_w16 = head.data.to(torch.bfloat16)
        else:
            self.head_grad = zeros(head.shape, torch.float32)
        # everything else keeps an ordinary, persistently allocated .grad; small ones share one flat buffer
        muon_ids = {id(p) for g in self.groups.values() for p in g.params}
        rest = [p for p in model.parameters() if id(p) not in muon_ids and p is not head]
        small = [p for p in rest if p.numel() < SMALL_NUMEL and p.dtype == torch.float32]
        self.small_params = small
        total = sum(p.numel() for p in small)
        self.small_P = torch.empty(total, dtype=torch.float32, device=dev)
        self.small_grads = zeros((max(total, 4),), torch.float32)[:total] if total > 0 else torch.zeros(0, device=dev)
        self.small_offsets = {}
        off = 0
        for p in small:
            n = p.numel()
            self.small_P[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.small_P[off:off + n].view_as(p)
            p.grad = self.small_grads[off:off + n].view_as(p)
            self.small_offsets[id(p)] = (off, n)
            off += n
        self.other_params = [p for p in rest if not (p.numel() < SMALL_NUMEL and p.dtype == torch.float32)]
        for p in self.other_params:
            repoint(p)
            p.grad = zeros(p.shape, p.dtype)
        if cuda and getattr(model, "wire_fused", True):
            self._wire_fused_views()

    # ------------------------------------------------------------------ fused operand views for the model
    def _slot(self, p):
        g = self.groups[tuple(p.shape)]
        return g, g.index_of(p)

    def _wire_fused_views(self):
        m = self.model
        for block in m.all_blocks():
            a = block.attn
            if getattr(a, "is_linear_attention", False):
                self._wire_mlp(block.mlp)
                continue
            g, iq = self._slot(a.c_q.weight)
            assert g.params[iq + 1] is a.c_k.weight and g.params[iq + 2] is a.c_v.weight, "q,k,v must be adjacent"
            d_out, d_in = g.shape
            g2, ip = self._slot(a.c_proj.weight)
            a.fused = dict(qkv_w16=g.W16[iq:iq + 3].view(3 * d_out, d_in), qkv_grad=g.G[iq:iq + 3].view(3 * d_out, d_in),
                           proj_w16=g2.W16[ip], proj_grad=g2.G[ip])
            self._wire_mlp(block.mlp)
        for lin in m.ve_projs.values():
            g, i = self._slot(lin.weight)
            lin.fused = dict(w16=g.W16[i], grad=g.G[i])
        if m.mtp_weight > 0:
            g, i = self._slot(m.mtp_proj.weight)
            m.mtp_proj.fused = dict(w16=g.W16[i], grad=g.G[i])

    def _wire_mlp(self, mlp):
        gg, ig = self._slot(mlp.c_gate.weight)
        assert gg.params[ig + 1] is mlp.c_fc.weight, "c_gate, c_fc must be adjacent"
        h, d = gg.shape
        g3, i3 = self._slot(mlp.c_proj.weight)
        mlp.fused = dict(gf_w16=gg.W16[ig:ig + 2].view(2 * h, d), gf_grad=gg.G[ig:ig + 2].view(2 * h, d),
                         proj_w16=g3.W16[i3], proj_grad=g3.G[i3])

    # ------------------------------------------------------------------ maintenance
    def zero_grads(self):
        for g in self.groups.values():
            g.G.zero_()
        self.head_grad.zero_()
        head = self.model.lm_head.weight
        if head.grad is not None and head.grad.data_ptr() != self.head_grad.data_ptr():
            head.grad = None          # autograd-made gradient of a bf16 head on the plain-PyTorch path
        self.small_grads.zero_()
        for p in self.other_params:
            p.grad.zero_()

    @torch.no_grad()
    def refresh_shadows(self):
        """Re-derive every bf16 shadow from its fp32 master (after loading a checkpoint or averaging weights)."""
        for g in self.groups.values():
            if g.W16 is not None:
                g.W16.copy_(g.P)
        if self.head_w16 is not None:
            self.head_w16.copy_(self.model.lm_head.weight.data)
