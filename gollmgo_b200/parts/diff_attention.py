"""Differential attention: every head has two attention maps over the same values, with query
and key projections of their own, and the head's result is their difference,

    o_h = A1_h V - lambda * A2_h V,        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff,

divided by its root mean square over the head's values and multiplied by (1 - diff).  lambda is
one number per layer, made of four learned vectors and the constant ``diff``.

A map is a softmax attention like any other, so the engine runs the 2H maps as 2H query heads
of size ``head_dim`` on 2G key heads, every two of which read one value head (the general
kernels' ``v_share``): keys are cached per map, values once.  Grouped-query attention needs
the query heads of one key head to lie together, so the rows of the query projection are
reordered at load time from [head][map] to [kv group][map][head in group]; the kernel that
combines the maps reads them in that order and writes heads in the checkpoint's order.

params: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, window, position (PartSpec),
scale, diff, eps, biases (bool), names (q, k, v, o), lambda_names (lq1, lk1, lq2, lk2), out_buffer,
defer_output_bias (bool: the output projection's bias is not added here but left in ``deferred_bias``
for a block that adds the mixer's result to the stream with a kernel that takes a bias).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .attention import Attention
from .linear import linear
from .registry import register_mixer


class DiffAttention(Attention):
    v_share = 2

    def __init__(self, spec, ctx):
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.bias = bool(spec.get("biases", False))
        self.diff = float(spec["diff"])
        self.eps = float(spec["eps"])
        self.lambda_names = tuple(spec.get("lambda_names") or ("lq1", "lk1", "lq2", "lk2"))
        self.defer_output_bias = bool(spec.get("defer_output_bias", False))
        self.deferred_bias = None
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        # the maps as heads: twice the heads on twice the key heads
        as_maps = dict(spec.params)
        as_maps["num_heads"], as_maps["num_kv_heads"] = 2 * self.heads, 2 * self.kv_heads
        as_maps.setdefault("names", ("q", "k", "v", "o"))
        super().__init__(type(spec)(spec.kind, as_maps), ctx)
        ctx.workspace.reserve("diff_maps", ctx.max_tokens * self.nh * self.dv, torch.float32)
        ctx.workspace.reserve("diff_heads", ctx.max_tokens * self.heads * self.dv, ctx.act_dtype)
        self.lam = None

    def weights(self):
        q, k, v, o = self.names
        w = {q: WeightSpec((self.nh * self.d, self.hidden)), k: WeightSpec((self.nkv * self.d, self.hidden)),
             v: WeightSpec((self.nv * self.dv, self.hidden)), o: WeightSpec((self.hidden, self.heads * self.dv))}
        if self.bias:
            w.update({q + ".b": WeightSpec((self.nh * self.d,), init="normal"),
                      k + ".b": WeightSpec((self.nkv * self.d,), init="normal"),
                      v + ".b": WeightSpec((self.nv * self.dv,), init="normal"),
                      o + ".b": WeightSpec((self.hidden,), init="normal")})
        w.update({n: WeightSpec((self.d,), init="normal") for n in self.lambda_names})
        return w

    def _by_group(self, t):
        """Rows [head][map][d] of a query tensor -> [kv group][map][head in group][d]."""
        rep = self.heads // self.kv_heads
        rest = t.shape[1:]
        return t.view(self.kv_heads, rep, 2, self.d, *rest).transpose(1, 2).reshape(self.nh * self.d, *rest).contiguous()

    def load(self, get):
        qn, kn, vn, on = self.names
        q, k, v = self._by_group(get(qn)), get(kn), get(vn)
        dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = get(on).contiguous()
        if self.bias:
            self.qkv_bias = torch.cat([self._by_group(get(qn + ".b")).float(), get(kn + ".b").float(),
                                       get(vn + ".b").float()]).contiguous()
            self.o_bias = get(on + ".b").float().contiguous()
            if self.defer_output_bias:
                self.deferred_bias = self.o_bias
        lq1, lk1, lq2, lk2 = (get(n).double() for n in self.lambda_names)
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff)

    def takes_normed_rows(self, num_tokens):
        return False

    def fuses_next_norm(self, num_tokens):
        return False

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        maps = self.attend_general(x, batch, cache, writes_cache, ws.get("diff_maps", T, self.nh * self.dv))
        heads = ws.get("diff_heads", T, self.heads * self.dv)
        ops.diff_combine(maps, heads, self.lam, self.eps, 1.0 - self.diff, self.heads, self.kv_heads, self.dv)
        y = linear(heads, self.w_o, ws.get(self.out_buffer, T, self.hidden))
        if self.o_bias is not None and not self.defer_output_bias:
            ops.bias_add(y, self.o_bias)
        return y


register_mixer("diff_attention", DiffAttention)
