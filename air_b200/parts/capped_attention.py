"""Grouped-query attention with the options that newer decoders add to it."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .attention import TiledAttention
from .base import Mixer, PagedKV
from .linear import Linear
from .registry import register_mixer, POSITION_ENCODINGS


@register_mixer("capped_attention")
class CappedAttention(TiledAttention, Mixer):
    """Causal softmax attention over the paged cache in which

      * keys and queries have one size per head (head_dim) and values another (v_dim);
      * the score is scale * q.k with `scale` given, and then softcap * tanh(score / softcap) where softcap > 0;
      * the position encoding may rotate only the first part of a head, at any position (its kernel takes the
        angles from the encoding's frequencies, in 32-bit);
      * values may be mixed across layers: the first layer of a `v_mix` stream hands its values of the step's tokens
        on (v_mix = "first"), a later one (v_mix = "mix") computes v = (1 - lambda) v + lambda v_first with a
        learned lambda, and the mixed values are what it caches;
      * each head's output may be multiplied by sigmoid of a logit of its own, projected from the layer's input
        (head_gate).

    params: hidden, heads, kv_heads, head_dim, v_dim, scale, softcap (0: none), window (None: all keys), qkv_bias,
    head_gate, v_mix (None, "first", "mix"), v_stream (the name under which the layers of a stream meet), position.
    Tensors: <prefix>q [heads*head_dim, hidden], k [kv_heads*head_dim, hidden], v [kv_heads*v_dim, hidden], each with
    <name>.b where qkv_bias; g [heads, hidden] where head_gate; vmix [] where v_mix; o [hidden, heads*v_dim].

    q, k, v and the gate are one product.  One kernel then adds the bias, rotates, mixes the values, writes keys and
    values to the pages and the gates to a small tensor.  In bfloat16, with keys and values of one size that the
    tensor-core attention kernels take (64 or 128; 256 for single tokens), those kernels attend, with the cap in their
    softmax, and a small kernel multiplies by the gates; otherwise the 32-bit attention kernel does all of it."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = p["hidden"], p["heads"], p["kv_heads"]
        self.head_dim, self.v_dim = p["head_dim"], p.get("v_dim") or p["head_dim"]
        self.scale, self.softcap = float(p["scale"]), float(p.get("softcap") or 0.0)
        self.window = p.get("window")
        self.qkv_bias, self.head_gate = bool(p.get("qkv_bias", False)), bool(p.get("head_gate", False))
        self.v_mix, self.v_stream = p.get("v_mix"), p.get("v_stream", "v_first")
        if self.v_mix not in (None, "first", "mix"):
            raise ConfigError("data_error", f"capped_attention: v_mix {self.v_mix!r}")
        if self.heads % self.kv_heads:
            raise ConfigError("data_error", "attention: heads must be a multiple of kv_heads")
        if max(self.head_dim, self.v_dim) > 256:
            raise ConfigError("unsupported", f"attention: head sizes {self.head_dim} / {self.v_dim}: the kernels take "
                                             "up to 256")
        pos = p["position"]
        self.position = POSITION_ENCODINGS.get(pos.kind)(pos)

    def cache_needs(self):
        return (PagedKV(self.kv_heads, self.head_dim, self.window, self.v_dim),)

    def plan_key(self):
        # (the tile kernels take keys and values of one size: other layers plan nothing)
        return TiledAttention.plan_key(self) if self.head_dim == self.v_dim else None

    def _names(self):
        return ["q", "k", "v"] + (["g"] if self.head_gate else [])

    def tensor_specs(self):
        p, e = self.prefix, self.hidden
        rows = {"q": self.heads * self.head_dim, "k": self.kv_heads * self.head_dim, "v": self.kv_heads * self.v_dim,
                "g": self.heads}
        specs = [TensorSpec(p + n, (rows[n], e)) for n in self._names()]
        if self.qkv_bias:
            specs += [TensorSpec(p + n + ".b", (rows[n],), wide=True) for n in "qkv"]
        if self.v_mix:
            specs.append(TensorSpec(p + "vmix", (), wide=True))
        specs.append(TensorSpec(p + "o", (e, self.heads * self.v_dim)))
        return specs + self.position.tensor_specs()

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        ws = [tensors[p + n] for n in self._names()]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{p}: the projections are stored in different precisions")
        self.proj = Linear(torch.cat(ws, dim=0).contiguous(), rt.status)
        self.o = Linear(tensors[p + "o"], rt.status)
        self.bias = None
        if self.qkv_bias:
            parts = [tensors[p + n + ".b"].to(torch.float32) for n in "qkv"]
            if self.head_gate:
                parts.append(torch.zeros(self.heads, dtype=torch.float32, device=rt.device))
            self.bias = torch.cat(parts).contiguous()
        self.v_lambda = tensors[p + "vmix"].to(torch.float32).reshape(1).contiguous() if self.v_mix == "mix" else None
        self.position.load(tensors, rt)
        if self.position.table() is not None:
            raise ConfigError("unsupported", "capped_attention takes a position encoding that gives frequencies")

    def forward(self, x, ctx, cache, owns_cache=True):
        if not owns_cache:
            raise ops.KernelError("capped_attention: a run that reads another run's keys and values is not offered")
        (pages,) = cache
        T, H, G, dk, dv = x.shape[0], self.heads, self.kv_heads, self.head_dim, self.v_dim
        rt = self.rt
        P = rt.page_tokens
        proj = self.proj.f32(x)
        q = torch.empty((T, H, dk), dtype=rt.dtype, device=x.device)
        gate = torch.empty((T, H), dtype=torch.float32, device=x.device) if self.head_gate else None
        v_mode, v_first = 0, None
        if self.v_mix == "first":
            v_mode = 1
            v_first = ctx.shared[self.v_stream] = torch.empty((T, G * dv), dtype=torch.float32, device=x.device)
        elif self.v_mix == "mix":
            v_mode, v_first = 2, ctx.shared.get(self.v_stream)
            if v_first is None:
                raise ops.KernelError(f"capped_attention: no earlier layer has handed on '{self.v_stream}'")
        bt = ctx.block_tables[pages.group]
        kv = pages.kv.view(pages.kv.shape[0], -1)
        ops.qkv_prepare(proj, self.bias, self.position.frequencies(), ctx.positions, ctx.token_seq, bt, q, kv, G, dv,
                        P, gate_out=gate, v_first=v_first, v_mode=v_mode, v_lambda=self.v_lambda, status=ctx.status)
        out = torch.empty((T, H, dv), dtype=rt.dtype, device=x.device)
        if dk == dv and self.fast_attention(ctx, P):
            self.attend(q, pages.kv, bt, ctx, out)
            if gate is not None:
                ops.head_gate(out, gate, ctx.token_seq)
        else:
            ops.paged_attention_ref(q, kv, bt, ctx.token_seq, ctx.positions, out, self.window, self.scale,
                                    softcap=self.softcap, gate=gate, kv_heads=G, page_tokens=P)
        return self.o.f32_sums(out.view(T, H * dv))
