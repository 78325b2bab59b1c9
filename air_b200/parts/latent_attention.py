"""Attention over a compressed latent: per token the cache holds one short row instead of keys and values per head."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Mixer, PagedLatent
from .gathered_attention import PortionAttention
from .linear import Linear
from .registry import register_mixer, POSITION_ENCODINGS


@register_mixer("latent_attention")
class LatentAttention(PortionAttention, Mixer):
    """q = Wq x, per head [head_dim plain | rot_dim rotated].  (c | kr) = Wdkv x: c (kv_rank columns) is normalised,
    c = rms(c) * w_c; kr (rot_dim columns) is one rotated key part for all heads.  Head h has the key [Wuk_h c | kr]
    and the value Wuv_h c; score = scale * (q_plain . Wuk_h c + q_rot . kr); causal softmax over the last `window` keys
    (None: all); output matrix on the concatenated heads.  Only the row [c | kr] is kept per token.

    The key and value expansions are never applied to the cache: q_plain is carried through Wuk_h once per query
    (q'_h = Wuk_h^T q_plain_h, so that q_plain . Wuk_h c = q'_h . c), every head then attends over the same rows [c | kr]
    with the query [q'_h | q_rot_h] and sums the rows' first kv_rank elements, and Wuv_h expands that sum.  The two
    small products per head are one grouped product each.

    params: hidden, heads, head_dim, rot_dim, v_dim, kv_rank, scale, window, eps, position (rope_live with rotary_dim =
    rot_dim), borrows (the layer has no Wdkv: its run reads the rows that another layer's run keeps), keep (the
    widest window among the layers that read this layer's rows: pages older than that go back to the pool).
    Tensors: <prefix>q [heads*(head_dim+rot_dim), hidden], dkv [kv_rank+rot_dim, hidden], dkv.norm [kv_rank],
    uk [heads*head_dim, kv_rank], uv [heads*v_dim, kv_rank], o [hidden, heads*v_dim]."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.head_dim = p["hidden"], p["heads"], p["head_dim"]
        self.rot_dim, self.v_dim, self.rank = p["rot_dim"], p["v_dim"], p["kv_rank"]
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 1e-6))
        self.window, self.borrows, self.chunk, self.sinks = p.get("window"), bool(p.get("borrows", False)), None, None
        self.keep = p.get("keep", self.window) if self.window else None
        if self.rank + self.rot_dim > 640:
            raise ConfigError("unsupported", f"latent attention: rows of {self.rank + self.rot_dim} numbers: the "
                                             "attention kernel takes up to 640")
        pos = p["position"]
        self.position = POSITION_ENCODINGS.get(pos.kind)(pos)

    def cache_needs(self):
        return () if self.borrows else (PagedLatent(self.rank + self.rot_dim, self.keep),)

    def tensor_specs(self):
        p, e, H = self.prefix, self.hidden, self.heads
        specs = [TensorSpec(p + "q", (H * (self.head_dim + self.rot_dim), e))]
        if not self.borrows:
            specs += [TensorSpec(p + "dkv", (self.rank + self.rot_dim, e)),
                      TensorSpec(p + "dkv.norm", (self.rank,), init="one_plus_normal", wide=True)]
        specs += [TensorSpec(p + "uk", (H * self.head_dim, self.rank)), TensorSpec(p + "uv", (H * self.v_dim, self.rank)),
                  TensorSpec(p + "o", (e, H * self.v_dim))]
        return specs + self.position.tensor_specs()

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p, H, d, R = self.prefix, self.heads, self.head_dim, self.rank
        q = tensors[p + "q"]
        self.c_weight = None
        if self.borrows:
            self.proj = Linear(q, rt.status)
        else:
            if tensors[p + "dkv"].dtype != q.dtype:
                raise ValueError(f"{p}: the projections are stored in different precisions")
            self.proj = Linear(torch.cat([q, tensors[p + "dkv"]], dim=0).contiguous(), rt.status)
            self.c_weight = tensors[p + "dkv.norm"].to(torch.float32).contiguous()
        # Wuk_h [d, R] is the product's [K, N]: the grouped product wants [N, K] per head
        self.uk_t = tensors[p + "uk"].view(H, d, R).transpose(1, 2).contiguous()
        self.uv = tensors[p + "uv"].view(H, self.v_dim, R).contiguous()
        self.o = Linear(tensors[p + "o"], rt.status)
        self.position.load(tensors, rt)
        if not hasattr(self.position, "frequencies64") or self.position.pairing != "half":
            raise ConfigError("unsupported", "latent attention takes a rotation in halves with 64-bit frequencies")
        if self.position.rotary_dim != self.rot_dim:
            raise ConfigError("data_error", "latent attention: the rotation covers the rotated part, all of it")

    def forward(self, x, ctx, cache, owns_cache=True):
        if owns_cache == self.borrows:
            raise ops.KernelError("latent attention: the layer and the run list disagree on whose rows the layer reads")
        (latent,) = cache
        T, H, d, rot, R, dv = x.shape[0], self.heads, self.head_dim, self.rot_dim, self.rank, self.v_dim
        rt = self.rt
        dev = x.device
        bt = ctx.block_tables[latent.group]
        proj = self.proj.f32(x)
        q_plain = torch.empty((T, H, d), dtype=rt.dtype, device=dev)
        q_full = torch.empty((T, H, R + rot), dtype=torch.float32, device=dev)
        ops.latent_prepare(proj, self.c_weight, self.eps, self.position.frequencies64(), ctx.positions, ctx.token_seq,
                           bt, q_plain, q_full, latent.rows, owns_cache, status=ctx.status)
        ops.grouped_gemm(q_plain, self.uk_t, q_full, R, d, lda=H * d, ldo=H * (R + rot), groups=H, a_group_stride=d,
                         o_group_stride=R + rot, a_local=True, o_local=True, rows_per_group=T)
        summed = torch.empty((T, H, R), dtype=rt.dtype, device=dev)
        self.attend(q_full, latent.rows, bt, ctx, summed, latent=True)
        out = torch.empty((T, H, dv), dtype=rt.dtype, device=dev)
        ops.grouped_gemm(summed, self.uv, out, dv, R, lda=H * R, ldo=H * dv, groups=H, a_group_stride=R,
                         o_group_stride=dv, a_local=True, o_local=True, rows_per_group=T)
        return self.o.f32_sums(out.view(T, H * dv))
