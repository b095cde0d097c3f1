"""The gated delta rule: a recurrent mixer whose state per head is a matrix S [d, dv],

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,

with q and k (``num_kv_heads`` heads of size ``head_dim``, shared by ``num_heads / num_kv_heads``
value heads each) and v (``num_heads`` heads of size ``v_head_dim``) passed through a short causal
convolution and SiLU, q and k made unit vectors (q times head_dim^-1/2), beta = sigmoid(Wb x),
g = exp(-exp(A_log) * softplus(Wa x + dt_bias)) per head.  The result is divided by its root mean
square per head, multiplied by a weight shared by the heads and by silu(Wg x), and projected.

State per request, in its state slot: S in float32 [heads, dv, d] and the last taps - 1 inputs
of the convolution in float32 [taps - 1, channels].  Nothing is paged.  Everything between the
projections and the output projection is float32 (csrc/delta_rule.cu).

params: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, conv (taps), eps, out_buffer,
names (optional dict: q, k, v, beta, a, gate, o, A_log, dt_bias, norm; the convolutions' tensors are
the q, k, v names + ".conv").
"""
from __future__ import annotations

import torch

from ..cache import FixedStateNeed
from ..csrc import ops
from ..weights import WeightSpec
from .linear import linear
from .registry import register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "beta": "b", "a": "a", "gate": "g", "o": "o", "A_log": "A_log",
          "dt_bias": "dt_bias", "norm": "norm"}


class GatedDeltaRule:
    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec["v_head_dim"])
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        self.names = dict(_NAMES, **(spec.get("names") or {}))
        self.out_buffer = spec.get("out_buffer") or "mixer_out"
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} q/k heads")
        if self.d > 256:
            raise ValueError(f"key size {self.d} is beyond what the recurrence kernel takes (256)")
        if not (1 <= self.taps <= 17):
            raise ValueError(f"{self.taps} taps are outside 1..17")
        self.channels = 2 * self.nkv * self.d + self.nh * self.dv            # q, k, v: what the convolution sees
        self.proj_width = self.channels + self.nh * self.dv                  # ... and the output gate
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("delta_proj", T * self.proj_width, ctx.act_dtype)
        ws.reserve("delta_ba", T * 2 * self.nh, torch.float32)
        ws.reserve("delta_qkv", T * self.channels, torch.float32)
        ws.reserve("delta_beta", T * self.nh, torch.float32)
        ws.reserve("delta_decay", T * self.nh, torch.float32)
        ws.reserve("delta_o", T * self.nh * self.dv, torch.float32)
        ws.reserve("delta_y", T * self.nh * self.dv, ctx.act_dtype)
        ws.reserve(self.out_buffer, T * self.hidden, ctx.act_dtype)
        self.w_proj = self.w_ba = self.w_o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def cache_need(self):
        need = [FixedStateNeed((self.nh, self.dv, self.d), "float32")]
        if self.taps > 1:
            need.append(FixedStateNeed((self.taps - 1, self.channels), "float32"))
        return tuple(need)

    def weights(self):
        n = self.names
        qk, vv = self.nkv * self.d, self.nh * self.dv
        w = {n["q"]: WeightSpec((qk, self.hidden)), n["k"]: WeightSpec((qk, self.hidden)),
             n["v"]: WeightSpec((vv, self.hidden)), n["gate"]: WeightSpec((vv, self.hidden)),
             n["beta"]: WeightSpec((self.nh, self.hidden)), n["a"]: WeightSpec((self.nh, self.hidden)),
             n["A_log"]: WeightSpec((self.nh,), init="normal"), n["dt_bias"]: WeightSpec((self.nh,), init="normal"),
             n["norm"]: WeightSpec((self.dv,)), n["o"]: WeightSpec((self.hidden, vv))}
        w.update({n["q"] + ".conv": WeightSpec((qk, self.taps), init="taps"),
                  n["k"] + ".conv": WeightSpec((qk, self.taps), init="taps"),
                  n["v"] + ".conv": WeightSpec((vv, self.taps), init="taps")})
        return w

    def load(self, get):
        n = self.names
        parts = [get(n[x]) for x in ("q", "k", "v", "gate")]
        dt = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_proj = torch.cat([p.to(dt) for p in parts], dim=0).contiguous()
        self.w_ba = torch.cat([get(n["beta"]), get(n["a"])], dim=0).contiguous()
        self.w_o = get(n["o"]).contiguous()
        self.conv_w = torch.cat([get(n[x] + ".conv").float() for x in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = get(n["A_log"]).float().contiguous()
        self.dt_bias = get(n["dt_bias"]).float().contiguous()
        self.norm_w = get(n["norm"]).float().contiguous()

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        state = cache[0]
        conv_state = cache[1] if self.taps > 1 else state        # unused without taps to carry
        proj = linear(x, self.w_proj, ws.get("delta_proj", T, self.proj_width))
        ba = linear(x, self.w_ba, ws.get("delta_ba", T, 2 * self.nh))
        qkv = ws.get("delta_qkv", T, self.channels)
        beta, decay = ws.get("delta_beta", T, self.nh), ws.get("delta_decay", T, self.nh)
        B = batch.num_seqs
        ops.delta_prep(proj, self.conv_w, conv_state, ba, self.a_log, self.dt_bias, batch.cu_q_lens, batch.context_lens,
                       batch.state_slots, B, self.nkv, self.nh, self.d, self.dv, qkv, beta, decay)
        o = ws.get("delta_o", T, self.nh * self.dv)
        ops.delta_recur(qkv, beta, decay, state, batch.cu_q_lens, batch.context_lens, batch.state_slots, B,
                        self.nkv, self.nh, self.d, self.dv, o)
        y = ws.get("delta_y", T, self.nh * self.dv)
        ops.delta_out(o, proj[:, self.channels:], self.norm_w, self.eps, self.nh, self.dv, y)
        return linear(y, self.w_o, ws.get(self.out_buffer, T, self.hidden), then)


register_mixer("gated_delta", GatedDeltaRule)
