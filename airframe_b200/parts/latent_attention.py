"""Attention whose keys and values are made from one small latent vector per
token, which is all the cache keeps.

Per token: [c' | r'] = W_dkv h with c' of ``kv_rank`` and r' of ``rot_dim``
elements; c = c' / rms(c') * w_norm is the latent, r = rotate(r') one rotated
key part that all heads share.  Head a has the key [W_uk,a c | r] and the value
W_uv,a c; its query q_a = W_q,a h is [``head_dim`` plain | ``rot_dim`` rotated]
elements.  score = (q_plain . k_plain + q_rot . r) * scale over a sliding
window, softmax (with a learned sink per head in the denominator when the
model has one), output projection over the concatenated heads.

The products with W_uk and W_uv are moved to the query's side, where they
cost one small product per new token instead of one per cached token:
q_plain . (W_uk,a c) = (W_uk,a^T q_plain) . c and sum_j p_j W_uv,a c_j =
W_uv,a (sum_j p_j c_j).  The attention itself then runs over one shared
key/value head whose key row is the cached [c | r] (``kv_rank + rot_dim``
elements) and whose value is the first ``kv_rank`` elements of the same row;
the cache holds no value pages.

A prompt in bfloat16 goes the other way round where the head sizes allow: one
product turns the step's rows [c | r] into every head's key [W_uk,a c | r] and
value W_uv,a c (the weight holds W_uk, W_uv and an identity for r, heads padded
with zeros up to a size the tensor-core attention kernels take), and those
kernels run as for ordinary heads; per token that costs a product with W_uk and
W_uv once, not once per key it sees.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError, PartSpec
from ..weights.loader import WeightDecl
from .base import KVNeed, Mixer, build_part, register_part
from .linear import linear, linear_split
from .rope import Rope


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (the plain part of a query/key head), ``rot_dim``
    (its rotated part), ``value_dim``, ``kv_rank``, ``scale``, ``window`` (None = all keys), ``mask`` ("window" or
    "chunk"), ``eps`` (of the latent's norm), ``position`` (a ``rope`` PartSpec with ``rotary_dim`` = ``rot_dim``
    and half-split pairs), tensor names ``q_weight`` [heads (head_dim + rot_dim), hidden], ``dkv_weight``
    [kv_rank + rot_dim, hidden], ``dkv_norm_weight`` [kv_rank], ``uk_weight`` [heads head_dim, kv_rank],
    ``uv_weight`` [heads value_dim, kv_rank], ``o_weight`` [hidden, heads value_dim]; optional ``sink_weight``
    [heads]; optional ``wide_output``."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dim = int(self.param("head_dim"))
        self.rot = int(self.param("rot_dim"))
        self.dv = int(self.param("value_dim"))
        self.rank = int(self.param("kv_rank"))
        self.scale = float(self.param("scale"))
        self.eps = float(self.param("eps"))
        w = self.params.get("window")
        self.window = int(w) if w else None
        self.mask = self.params.get("mask") or "window"
        if self.mask not in kernels.MASKS:
            raise ConfigError(f"latent_attention: unknown mask '{self.mask}'")
        if self.dim < 1 or self.rot % 2:
            raise ConfigError(f"latent_attention: head_dim {self.dim} must be positive and rot_dim {self.rot} even")
        self.position = build_part("position", self.param("position"), ctx)
        if not isinstance(self.position, Rope) or self.position.pairing != "half" or self.position.rotary_dim != self.rot \
                or self.position.magnitude != 1.0:
            raise ConfigError("latent_attention: the position encoding is a plain rotation of half-split pairs over rot_dim")
        self.names = {k: self.param(k) for k in ("q_weight", "dkv_weight", "dkv_norm_weight", "uk_weight", "uv_weight",
                                                 "o_weight")}
        self.sink_name = self.params.get("sink_weight")
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.norm_w = self.sinks = None
        self.fast_hd = 0            # head size of the prompt's tensor-core path (0: there is none)
        self.w_up = self.w_o_fast = None

    def kv_need(self):
        return KVNeed(1, self.rank + self.rot, self.window, 0)       # (values: the latent part of the key row)

    def weight_decls(self):
        n, H, h = self.names, self.heads, self.hidden
        decls = [WeightDecl(n["q_weight"], (H * (self.dim + self.rot), h)),
                 WeightDecl(n["dkv_weight"], (self.rank + self.rot, h)),
                 WeightDecl(n["dkv_norm_weight"], (self.rank,), "norm"),
                 WeightDecl(n["uk_weight"], (H * self.dim, self.rank)),
                 WeightDecl(n["uv_weight"], (H * self.dv, self.rank)),
                 WeightDecl(n["o_weight"], (h, H * self.dv))]
        if self.sink_name:
            decls.append(WeightDecl(self.sink_name, (H,), "norm"))
        return [*decls, *self.position.weight_decls()]

    def load(self, weights):
        n, dt, H = self.names, self.ctx.compute_dtype, self.heads
        # one product for the queries and the latent: rows [q heads | latent | shared key part]
        self.w_in = torch.cat([weights[n["q_weight"]], weights[n["dkv_weight"]]], dim=0).to(dt).contiguous()
        # per head: q_plain [dim] -> rank (W_uk as it lies), weighted latent [rank] -> value_dim (W_uv transposed)
        self.w_uk = weights[n["uk_weight"]].to(dt).reshape(H, self.dim, self.rank).contiguous()
        self.w_uv = weights[n["uv_weight"]].to(dt).reshape(H, self.dv, self.rank).transpose(1, 2).contiguous()
        self.w_o = weights[n["o_weight"]].to(dt).contiguous()
        self.norm_w = weights[n["dkv_norm_weight"]].to(torch.float32).contiguous()
        if self.sink_name:
            self.sinks = weights[self.sink_name].to(torch.float32).contiguous()
        self.position.load(weights)
        # a prompt's path over the tensor-core attention kernels: keys and values of every head out of one product
        hd = 0
        if dt == torch.bfloat16 and self.w_o.is_cuda and (self.rank + self.rot) % 8 == 0 and self.mask == "window":
            hd = kernels.attn_prefill_fast_head(max(self.dim + self.rot, self.dv))
        if hd:
            up = torch.zeros(2 * H * hd, self.rank + self.rot, dtype=dt, device=self.w_o.device)
            k_rows, v_rows = up[: H * hd].view(H, hd, -1), up[H * hd:].view(H, hd, -1)
            k_rows[:, : self.dim, : self.rank] = weights[n["uk_weight"]].to(dt).view(H, self.dim, self.rank)
            k_rows[:, self.dim: self.dim + self.rot, self.rank:] = torch.eye(self.rot, dtype=dt, device=up.device)
            v_rows[:, : self.dv, : self.rank] = weights[n["uv_weight"]].to(dt).view(H, self.dv, self.rank)
            self.w_up = up
            if hd == self.dv:
                self.w_o_fast = self.w_o
            else:
                wide = torch.zeros(self.hidden, H, hd, dtype=dt, device=up.device)
                wide[:, :, : self.dv] = self.w_o.view(self.hidden, H, self.dv)
                self.w_o_fast = wide.view(self.hidden, H * hd).contiguous()
            self.fast_hd = hd

    def _el(self) -> int:
        return 4 if self.ctx.compute_dtype == torch.float32 else 2

    def _visible(self, pos: int) -> int:
        if not self.window:
            return pos + 1
        return pos % self.window + 1 if self.mask == "chunk" else min(pos + 1, self.window)

    def decode_bytes(self, lens) -> int:
        weights = (self.w_in.numel() + self.w_uk.numel() + self.w_uv.numel() + self.w_o.numel()) * self._el()
        return weights + sum((self.rank + self.rot) * self._el() * self._visible(n - 1) for n in lens)

    def score_flops(self, lens) -> int:
        """Scores and weighted sums over the latent rows, as this part computes them."""
        pairs = 0
        for n in lens:
            w = self.window
            if w and self.mask == "chunk":
                full, rest = divmod(n, w)
                pairs += full * (w * (w + 1) // 2) + rest * (rest + 1) // 2
            else:
                pairs += n * (n + 1) // 2 if not w or n <= w else w * (w + 1) // 2 + (n - w) * w
        if self.fast_hd:        # (a prompt's path: ordinary heads of dim + rot key and value_dim value elements)
            return 2 * pairs * self.heads * (self.dim + self.rot + self.dv)
        return 2 * pairs * self.heads * (2 * self.rank + self.rot)

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        proj = 2 * T * (self.w_in.numel() + self.w_uk.numel() + self.w_uv.numel() + self.w_o.numel())
        return proj + self.score_flops(lens)

    FAST_PROMPT_ROWS = 64      # from this many rows on a bfloat16 prompt takes the tensor-core path

    def _prompt_on_tensor_cores(self, proj, batch, view):
        """Keys and values of every head from the step's latent rows by one product, then the attention kernels
        of ordinary heads (a window, a sink)."""
        H, hd = self.heads, self.fast_hd
        T, dt, dev = proj.shape[0], self.ctx.compute_dtype, proj.device
        q = torch.empty(T, H * hd, dtype=dt, device=dev)
        kvrow = torch.empty(T, self.rank + self.rot, dtype=dt, device=dev)
        kernels.latent_prep(q, kvrow, proj, batch, H, self.dim, self.rot, self.rank, self.norm_w, self.eps,
                            self.position.inv_freq, kv=view.kv if view.writes else None, pitch=hd)
        if not view.writes:
            kvrow = batch.step_kv[view.cache_id][0]
        elif view.keep_step_kv:
            batch.step_kv[view.cache_id] = (kvrow, kvrow[:, : self.rank])
        kv_up = linear(kvrow, self.w_up)
        ctx = torch.empty(T, H * hd, dtype=dt, device=dev)
        kernels.attn_prefill(ctx, q, kv_up[:, : H * hd], kv_up[:, H * hd:], batch, H, H, hd, self.scale, 0.0,
                             self.window or 0, mask=self.mask, sinks=self.sinks)
        return linear_split(ctx, self.w_o_fast, wide=bool(self.params.get("wide_output", False)))

    def forward(self, x, batch, view):
        H, dim, rot, rank, dv = self.heads, self.dim, self.rot, self.rank, self.dv
        T, dt = x.shape[0], x.dtype
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        if batch.is_prefill and self.fast_hd and T >= self.FAST_PROMPT_ROWS:
            return self._prompt_on_tensor_cores(proj, batch, view)
        q = torch.empty(T, H * (dim + rot), dtype=dt, device=x.device)
        kvrow = torch.empty(T, rank + rot, dtype=dt, device=x.device)
        kernels.latent_prep(q, kvrow, proj, batch, H, dim, rot, rank, self.norm_w, self.eps, self.position.inv_freq,
                            kv=view.kv if view.writes else None)
        # the queries on the latent's side: [W_uk^T q_plain | q_rot] per head
        q_lat = torch.empty(T, H * (rank + rot), dtype=dt, device=x.device)
        kernels.head_project(q_lat, q, self.w_uk, H, dim, rank, extra=rot)
        # a decode step whose key rows have a size the split kernel takes gets whole rows [sum p c | sum p r] back
        # from it (the key pages serve as value pages); the values' part is read from there
        wide = not batch.is_prefill and kernels.attn_decode_fast(dt, rank + rot, batch.n_seqs)
        mix = torch.empty(T, H * (rank + rot if wide else rank), dtype=dt, device=x.device)
        window = self.window or 0
        if batch.is_prefill:
            if not view.writes:
                kvrow = batch.step_kv[view.cache_id][0]
            elif view.keep_step_kv:
                batch.step_kv[view.cache_id] = (kvrow, kvrow[:, :rank])
            kernels.attn_prefill(mix, q_lat, kvrow, kvrow[:, :rank], batch, H, 1, rank + rot, self.scale, 0.0, window,
                                 dv=rank, mask=self.mask, sinks=self.sinks)
        else:
            kernels.attn_decode(mix, q_lat, view.kv, batch, H, 1, rank + rot, self.scale, 0.0, window, dv=rank,
                                mask=self.mask, sinks=self.sinks)
        # back from the latent to the heads' values, then the output projection
        ctx = torch.empty(T, H * dv, dtype=dt, device=x.device)
        kernels.head_project(ctx, mix, self.w_uv, H, rank, dv, x_pitch=rank + rot if wide else rank)
        return linear_split(ctx, self.w_o, wide=bool(self.params.get("wide_output", False)))
