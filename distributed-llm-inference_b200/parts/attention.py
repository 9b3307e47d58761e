"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import torch

from ..cache.needs import PagedKVNeed
from ..kernels import attention as attn_kernels
from ..kernels import ops
from ..kernels.gemm import last_product, project
from ..weights.loader import TensorDecl
from .base import Part, build_part, register_part, tensor_name


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q, k, v projections, position encoding, causal attention of each token over the keys of
    its own sequence at positions <= its own (optionally only the last ``window``), output
    projection (src/dli/model/llama.py:72-76,94-95,147-177).  Query head h reads kv head
    h // (num_heads / num_kv_heads).  The three projection matrices are read by their own
    names and laid side by side at load, so one product yields q | k | v.

    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window, position (PartSpec).
    """

    graph_capturable = True
    takes_scaled_rows = True  # the input only goes to the q | k | v product
    defer_output = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.nh % self.nkv:
            raise ValueError(f"num_heads={self.nh} is not a multiple of num_kv_heads={self.nkv}")
        self.position = build_part("position", p["position"], env)
        self.wqkv: torch.Tensor | None = None
        self.wo: torch.Tensor | None = None

    def children(self):
        return [self.position]

    def declare(self):
        px, H, d = self.spec.prefix, self.hidden, self.d
        return {
            px + "q_proj.weight": TensorDecl((self.nh * d, H)),
            px + "k_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "v_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "o_proj.weight": TensorDecl((H, self.nh * d)),
        }

    def load(self, tensors):
        px = self.spec.prefix
        self.wqkv = torch.cat([tensors[px + "q_proj.weight"], tensors[px + "k_proj.weight"], tensors[px + "v_proj.weight"]], 0).contiguous()
        self.wo = tensors[px + "o_proj.weight"]

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        """Into how many runs the decode kernel cuts each sequence's keys (1: not at all)."""
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.d, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        encode = getattr(self.position, "project_and_encode", None)
        if encode is not None:  # the position part may fuse the projection with its encoding
            q = encode(x, self.wqkv, batch, cache, self.nh, self.nkv, cache.writes)
        else:
            q = self.position.rotate_and_store(project(x, self.wqkv), batch, cache, self.nh, self.nkv, cache.writes)
        out = torch.empty((x.shape[0], self.nh * self.d), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)))
        return last_product(out, self.wo, self.defer_output)


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    """Causal grouped-query attention whose softmax has a sink, with options other designs can switch:

    * ``sink`` (a score, or None): exp(sink) is added to every softmax denominator and carries no value,
      p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)), so a token may attend to nothing;
    * ``qk_norm_eps`` (or None): q and k are each divided by the RMS of their whole projection (all heads
      together, before they are cut into heads) and multiplied by a weight of that size, before the position
      encoding;
    * ``values``: ``"keys"`` — the values are the keys as projected (before norm and rotation; no value matrix)
      — or ``"projected"`` (a value matrix of its own);
    * ``gate``: the concatenated heads are multiplied by sigmoid(Wg x) before the output projection.

    One product yields q | k (| v) (| g); one kernel norms, rotates and writes the cache (the position part's
    ``norm_rotate_and_store``); the framework's attention kernels run with their sink argument.
    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window, position (PartSpec), sink,
    qk_norm_eps, values, gate, tensors (names of q, k, v, g, o, q_norm, k_norm)."""

    graph_capturable = True
    takes_scaled_rows = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.sink = None if p.get("sink") is None else float(p["sink"])
        self.qk_norm_eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.values_from_keys = p.get("values", "projected") == "keys"
        self.gated = bool(p.get("gate", False))
        if p.get("values", "projected") not in ("keys", "projected"):
            raise ValueError(f"values={p['values']!r} (keys, projected)")
        if self.nh % self.nkv:
            raise ValueError(f"num_heads={self.nh} is not a multiple of num_kv_heads={self.nkv}")
        self.position = build_part("position", p["position"], env)
        if not hasattr(self.position, "norm_rotate_and_store"):
            raise ValueError(f"position part {p['position'].kind!r} cannot follow a norm over the whole projection")
        self.names = {role: tensor_name(spec, role, default) for role, default in (
            ("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("g", "g_proj.weight"), ("o", "o_proj.weight"),
            ("q_norm", "q_norm.weight"), ("k_norm", "k_norm.weight"))}
        self.w_in: torch.Tensor | None = None
        self.wo: torch.Tensor | None = None
        self.wq_norm = self.wk_norm = None
        self.gate_col = (self.nh + (1 if self.values_from_keys else 2) * self.nkv) * self.d

    def children(self):
        return [self.position]

    def declare(self):
        H, d, nm = self.hidden, self.d, self.names
        out = {nm["q"]: TensorDecl((self.nh * d, H)), nm["k"]: TensorDecl((self.nkv * d, H)), nm["o"]: TensorDecl((H, self.nh * d))}
        if not self.values_from_keys:
            out[nm["v"]] = TensorDecl((self.nkv * d, H))
        if self.gated:
            out[nm["g"]] = TensorDecl((self.nh * d, H))
        if self.qk_norm_eps is not None:
            out[nm["q_norm"]] = TensorDecl((self.nh * d,), "vector32")
            out[nm["k_norm"]] = TensorDecl((self.nkv * d,), "vector32")
        return out

    def load(self, tensors):
        nm = self.names
        rows = [tensors[nm["q"]], tensors[nm["k"]]]
        if not self.values_from_keys:
            rows.append(tensors[nm["v"]])
        if self.gated:
            rows.append(tensors[nm["g"]])
        self.w_in = torch.cat(rows, 0).contiguous()
        self.wo = tensors[nm["o"]]
        if self.qk_norm_eps is not None:
            self.wq_norm, self.wk_norm = tensors[nm["q_norm"]], tensors[nm["k_norm"]]

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.d, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        proj = project(x, self.w_in)
        q = self.position.norm_rotate_and_store(proj, self.wq_norm, self.wk_norm, self.qk_norm_eps or 0.0, batch, cache, self.nh, self.nkv,
                                                cache.writes, self.values_from_keys)
        out = torch.empty((x.shape[0], self.nh * self.d), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)),
                                     sink=self.sink)
        if self.gated:
            ops.sigmoid_gate(out, proj[:, self.gate_col : self.gate_col + self.nh * self.d])
        return project(out, self.wo)
