"""Attention whose keys and values are linear maps of one latent row per token.

    c_q = norm(W_dq h; g_q)                 q = W_uq c_q        per head [dim unrotated | rot_dim rotated]
    [c' | k_r] = W_dkv h                    c = norm(c'; g_kv)  (k_r is not normed; it is rotated and shared by all heads)
    k_h = W_uk,h c     v_h = W_uv,h c       score_h(t, j) = (q_h . k_h,j + rot(q_r,h) . rot(k_r,j)) * scale
    softmax over the causal window, o = W_o (concat_h(sum_j p_j v_h,j) * sigmoid(W_g h))

Only c and the rotated k_r are cached: one row of `kv_rank + rot_dim` numbers per token for all
heads (`KVNeed` with one kv head and no value pool).  Keys and values are never expanded per
cached token: the per-head maps go to the query's side, (W_uk,h^T q_h) . c_j and W_uv,h (sum_j p_j c_j),
so the attention is multi-query attention over the latent rows (`csrc/latent_attn.cu`), for
prompts, portions and single tokens alike.

Norms, angles, scores and the softmax are 32-bit; in bfloat16 runs the projections' outputs that
feed a norm or the attention stay 32-bit rows (wide queries, latent means), the cache rows are
bfloat16.  Options: `window` (None: all earlier tokens), `gate` (None or "sigmoid"), a position
part for the rotated part (None: it is used as it comes).
"""
from __future__ import annotations

import torch

from ..kernels import attention as attention_kernels
from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import KVNeed, Mixer, Runtime, StepContext
from .registry import make_part, register_part
from .spec import PartSpec

DEFAULT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                 "g": "g", "o": "o"}

MIN_KEYS_PER_SLICE = 128      # single tokens: a slice of a row's keys shorter than this is not worth a block


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    returns_branch = True

    @property
    def kernel_libraries(self):
        return ("latent_attn", "latent_attn_tc", "grouped_gemm") if self.runtime.dtype == torch.bfloat16 else ("latent_attn",)

    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, scale: float, eps: float, position: PartSpec | None = None,
                 window: int | None = None, gate: str | None = None, names: dict | None = None):
        if gate not in (None, "sigmoid"):
            raise ValueError(f"latent_attention: gate {gate!r} is not supported (supported: 'sigmoid')")
        if kv_rank > 1024:
            raise ValueError(f"latent_attention: a latent of {kv_rank} numbers exceeds 1024")
        self.runtime, self.D, self.H = runtime, hidden_size, n_heads
        self.dn, self.dr, self.dv, self.Rq, self.R = head_dim, rot_dim, value_dim, q_rank, kv_rank
        self.scale, self.eps, self.window, self.gate = float(scale), float(eps), window, gate
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.position = make_part("position", position, runtime) if (position is not None and rot_dim) else None
        self.rot = getattr(self.position, "rotary_dims", rot_dim) if self.position is not None else 0
        self.w_dq: linear.LinearWeight | None = None
        self.w_down: linear.LinearWeight | None = None
        self.w_uq: linear.LinearWeight | None = None
        self.w_o: linear.LinearWeight | None = None
        self.w_uk = self.w_uv = self.w_uk_t = self.w_uv_t = self.g_q = self.g_kv = None
        self.tc_heads = False

    def cache_need(self):
        return KVNeed(1, self.R + self.dr, self.window, values=False)

    def step_needs(self):
        """The tensor-core kernel's work list for steps with prompts: blocks of consecutive tokens of one sequence."""
        if self.runtime.dtype != torch.bfloat16 or (self.R + self.dr) % 8:
            return {}
        size = ops.latent_tc_tokens(self.H)
        return {f"latent_blocks{size}": attention_kernels.query_blocks(size)}

    def weights(self):
        n, H = self.names, self.H
        out = {n["dq"]: WeightSpec((self.Rq, self.D)), n["dq_norm"]: WeightSpec((self.Rq,), init="gain", full_precision=True),
               n["uq"]: WeightSpec((H * (self.dn + self.dr), self.Rq)),
               n["dkv"]: WeightSpec((self.R + self.dr, self.D)),
               n["dkv_norm"]: WeightSpec((self.R,), init="gain", full_precision=True),
               n["uk"]: WeightSpec((H * self.dn, self.R)), n["uv"]: WeightSpec((H * self.dv, self.R)),
               n["o"]: WeightSpec((self.D, H * self.dv))}
        if self.gate is not None:
            out[n["g"]] = WeightSpec((H * self.dv, self.D))
        return out

    def load(self, tensors):
        n, H = self.names, self.H
        rows = [tensors[n["dkv"]]] + ([tensors[n["g"]]] if self.gate is not None else [])
        if len({r.dtype for r in rows}) > 1:
            rows = [r.to(torch.float32) for r in rows]
        # Two products from the layer's input: the query's bottleneck; the latent with the shared key part and the gate.
        self.w_dq = linear.LinearWeight(tensors[n["dq"]])
        self.w_down = linear.LinearWeight(torch.cat(rows, dim=0))
        self.w_uq = linear.LinearWeight(tensors[n["uq"]])
        self.w_o = linear.LinearWeight(tensors[n["o"]])
        self.g_q = tensors[n["dq_norm"]].to(torch.float32).contiguous()
        self.g_kv = tensors[n["dkv_norm"]].to(torch.float32).contiguous()
        # Per head: W_uk,h as stored is [dim, R] = [K, N] for q -> latent; W_uv,h [vdim, R] is turned to [R, vdim].
        self.w_uk = tensors[n["uk"]].reshape(H, self.dn, self.R).contiguous()
        self.w_uv = tensors[n["uv"]].reshape(H, self.dv, self.R).transpose(1, 2).contiguous()
        # The tensor-core products read every head's matrix as [outputs, inputs].
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()
        self.w_uv_t = tensors[n["uv"]].reshape(H, self.dv, self.R).contiguous()
        self.tc_heads = (self.runtime.dtype == torch.bfloat16 and self.w_uk.dtype == torch.bfloat16 and self.dn % 8 == 0
                         and (self.dn + self.dr) % 8 == 0 and self.R % 8 == 0)

    def _splits(self, ctx: StepContext, blocks_per_token: int, places_per_sm: int = 1) -> int:
        """Slices per row for a step of single tokens: as many as fill the multiprocessors, none shorter than
        MIN_KEYS_PER_SLICE.  A fixed number per batch size (the step may be captured and replayed)."""
        if not ctx.decode:
            return 1
        reach = min(self.window or self.runtime.max_context, self.runtime.max_context)
        blocks = max(ctx.T * blocks_per_token, 1)
        return max(1, min(places_per_sm * ops.sm_count(self.runtime.device) // blocks, reach // MIN_KEYS_PER_SLICE, 32))

    def _attend(self, wide, pages, ctx: StepContext, cache_view):
        """The weighted means of latent rows [T, H, R]: on the tensor cores where the cache allows it (bfloat16 rows out
        where the per-head products that follow run there too), else float32."""
        H, R = self.H, self.R
        more = {"out_dtype": torch.bfloat16} if self.tc_heads else {}
        if ops.latent_attention_tc_takes(pages, cache_view.page_size):
            chunks = -(-R // 512) if R > 256 else 1          # blocks along the value columns (two chunks of 256 share a block)
            if ctx.decode:
                return ops.latent_attention_tc(wide, pages, cache_view.page_table, ctx.slots, H, R, cache_view.page_size,
                                               self.scale, self.window, tok_pos=ctx.tok_pos, tok_seq=ctx.tok_seq,
                                               splits=self._splits(ctx, -(-H // 64) * chunks), **more)
            flat = ctx.extra.get(f"latent_blocks{ops.latent_tc_tokens(H)}")
            if flat is not None and flat.numel():
                return ops.latent_attention_tc(wide, pages, cache_view.page_table, ctx.slots, H, R, cache_view.page_size,
                                               self.scale, self.window, blocks=tuple(flat.view(4, -1)), **more)
        return ops.latent_attention(wide, pages, cache_view.page_table, ctx.tok_pos, ctx.tok_seq, ctx.slots, H, R,
                                    cache_view.page_size, self.scale, self.window, self._splits(ctx, -(-H // 8)))

    def forward(self, h, ctx: StepContext, cache_view, residual, writes_cache: bool = True):
        if not writes_cache:
            raise ValueError("latent_attention: the layer writes its own cache entry")
        H, dn, dr, dv, R, Rq = self.H, self.dn, self.dr, self.dv, self.R, self.Rq
        act = self.runtime.act_dtype
        T = h.shape[0]
        cq = ops.rmsnorm(linear.linear(h, self.w_dq, torch.float32), self.g_q, self.eps, act)      # norms read 32-bit sums
        down = linear.linear(h, self.w_down, torch.float32)          # [T, R + dr (+ H dv)]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        pages = cache_view.k_pages[:, 0]                             # one kv head: [pages, page_size, R + dr]
        ops.latent_kv_store(down, 0, R, self.g_kv, self.eps, cos, sin, self.rot, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                            cache_view.page_table, pages, R, dr, cache_view.page_size)
        q = linear.linear(cq, self.w_uq, act if self.tc_heads else torch.float32)     # [T, H (dn + dr)]
        wide = torch.empty((T, H, R + dr), dtype=torch.float32, device=q.device)
        wide2 = wide.view(T, H * (R + dr))
        if self.tc_heads and ops.grouped_gemm_takes(q, self.w_uk_t, dn + dr):
            ops.grouped_gemm(q, self.w_uk_t, wide2, a_group_stride=dn + dr, o_group_stride=R + dr)      # W_uk,h^T q_h
        else:
            ops.head_matmul(q, dn + dr, 0, self.w_uk, wide2, R + dr, 0)
        ops.rope_tail(q, dn + dr, dn, wide2, R + dr, R, cos, sin, self.rot, ctx.tok_pos, H, dr)
        mean = self._attend(wide, pages, ctx, cache_view)
        out = torch.empty((T, H * dv), dtype=act, device=q.device)
        mean = mean.view(T, H * R)
        if mean.dtype == torch.bfloat16 and ops.grouped_gemm_takes(mean, self.w_uv_t, R):
            ops.grouped_gemm(mean, self.w_uv_t, out, a_group_stride=R, o_group_stride=dv)                  # W_uv,h (sum_j p_j c_j)
        else:
            ops.head_matmul(mean, R, 0, self.w_uv, out, dv, 0)
        if self.gate is not None:
            ops.gate_mul(out, down[:, R + dr:], "sigmoid")
        if residual is None:
            return linear.linear(out, self.w_o, torch.float32)
        linear.linear(out, self.w_o, self.runtime.act_dtype, residual=residual)
        return None
