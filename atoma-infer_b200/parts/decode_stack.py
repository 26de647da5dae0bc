"""A run of whole layers of a decode step as one kernel launch.

Blocks say what they are made of (``Block.decode_fusion``); consecutive runs of the schedule whose blocks are the
arrangement the kernel knows (pre-norm residual block of RMSNorm, rotary attention over a paged cache and SwiGLU), with
equal sizes and the same cache group, become a ``DecodeStack``.  A decode step of at most 16 rows then runs the stack
instead of the blocks' own ``forward``; every other step, and every block that says nothing of itself, runs part by
part.  The blocks stay what they are: the stack only reads their bound tensors and constants.

The reference runs a layer as about 25 library kernels (models/src/llama.rs:259-410).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

MAX_ROWS = 16


def _geometry(f: Dict[str, Any]) -> Optional[Tuple]:
    """What must be equal along a stack; None: not an arrangement the kernel knows."""
    if f.get("kind") != "prenorm":
        return None
    n1, mx, n2, ff = f["norm1"], f["mixer"], f["norm2"], f["feed_forward"]
    if (n1.get("kind"), mx.get("kind"), n2.get("kind"), ff.get("kind")) != ("rmsnorm", "attention", "rmsnorm", "swiglu"):
        return None
    if n1["eps"] != n2["eps"] or not (n1["size"] == n2["size"] == mx["hidden"] == ff["hidden"]):
        return None
    if any(t.dtype != torch.bfloat16 for t in (mx["w_qkv"], mx["w_o"], ff["w_gate_up"], ff["w_down"])):
        return None
    return (mx["hidden"], mx["num_heads"], mx["num_kv_heads"], mx["head_dim"], float(mx["scale"]), mx["window"],
            mx["rotary_dim"], float(n1["eps"]), ff["intermediate"])


class DecodeStack:
    """Runs ``first`` .. ``end - 1`` of the schedule, bound and ready to launch."""

    def __init__(self, first: int, fusions: Sequence[Dict[str, Any]], group: int, rt):
        self.first, self.end = first, first + len(fusions)
        self.fusions, self.group, self.rt = list(fusions), group, rt
        (self.hidden, self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window, self.rotary_dim, self.eps,
         self.intermediate) = _geometry(fusions[0])
        self._table = None     # the layers' descriptors on the device, and the cache they were made for
        self._table_key = None
        self.arrivals = torch.zeros(1, dtype=torch.int64, device=rt.device)  # the kernel's grid barrier counts here

    def supports(self, rows: int) -> bool:
        # the kernel's tensor maps see every matrix in groups of 64 along k
        if self.hidden % 64 or self.intermediate % 64 or (self.num_heads * self.head_dim) % 64:
            return False
        return self.rt.ops.decode_stack_blocks(self.head_dim, rows, max(self.hidden, self.num_heads * self.head_dim)) > 0

    def _layer_table(self, views) -> torch.Tensor:
        key = tuple((v.pages.data_ptr(), bool(v.writes)) for v in views)
        if key != self._table_key:
            layers = []
            for f, v in zip(self.fusions, views):
                mx, ff = f["mixer"], f["feed_forward"]
                layers.append(dict(w_qkv=mx["w_qkv"], w_o=mx["w_o"], w_gate_up=ff["w_gate_up"], w_down=ff["w_down"],
                                   norm1=f["norm1"]["weight"], norm2=f["norm2"]["weight"], inv_freq=mx["inv_freq"],
                                   cache=v.pages, store_kv=bool(v.writes)))
            self._table = self.rt.ops.decode_stack_layers(layers, d=self.head_dim, hidden=self.hidden,
                                                          intermediate=self.intermediate, nq=self.num_heads,
                                                          nkv=self.num_kv_heads, page_size=views[0].page_size,
                                                          num_pages=views[0].num_pages)
            self._table_key = key
        return self._table

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, views) -> None:
        """resid += every layer's additions (and ``delta`` first); nothing is left pending."""
        v0 = views[0]
        self.rt.ops.decode_stack(self._layer_table(views), len(self.fusions), resid, delta, self.arrivals, ctx, self.group,
                                 hidden=self.hidden, intermediate=self.intermediate, nq=self.num_heads, nkv=self.num_kv_heads,
                                 d=self.head_dim, rot=self.rotary_dim, window=self.window, page_size=v0.page_size,
                                 num_pages=v0.num_pages, eps=self.eps, scale=self.scale,
                                 all_store_kv=all(v.writes for v in views))


    # ------------------------------------------------------------------ the chain: a kernel per linear, no norm kernels
    def chain_supports(self, rows: int) -> bool:
        """Whether a decode step of ``rows`` rows runs this stretch as a chain of streamed linears with the norms folded
        into them: wherever the kernels' policy streams every linear of the layer."""
        ops = self.rt.ops
        # measured, Llama 3.2 1B sizes, ms a decode step without / with the norms folded in: batch 2: 0.793 / 0.763;
        # batch 8: 0.831 / 0.826; batch 16 (two n-tiles, a heavier epilogue): 0.953 / 0.978
        if not getattr(ops, "fold_norms", False) or not hasattr(ops, "linear_streamed") or len(self.fusions) == 0 or rows > 8:
            return False
        qkv_rows = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        shapes = [(qkv_rows, self.hidden), (self.hidden, self.num_heads * self.head_dim), (2 * self.intermediate, self.hidden),
                  (self.hidden, self.intermediate)]
        return all(ops._stream_linear(rows, n, k) for n, k in shapes)

    def forward_chain(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, views) -> None:
        """The stretch's layers on a decode step, a launch per linear and one for the attention.  Only the first norm is a
        kernel of its own; every other norm is folded into the linears around it: the output and down projections add
        into the residual and leave the next linear's x (residual times the next norm's weight) and the rows' sums of
        squares, and the q/k/v and gate/up projections scale their rows by the 1 / rms those sums give.  The last down
        projection only adds into the residual: the model's final norm follows as usual."""
        ops, T = self.rt.ops, ctx.T
        first = self.fusions[0]["norm1"]
        x = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=resid.device)
        ops.add_rmsnorm(resid, delta, first["weight"], first["eps"], x, ctx.meta, T)
        scale = None
        for i, (f, view) in enumerate(zip(self.fusions, views)):
            mx, ff = f["mixer"], f["feed_forward"]
            qkv = ops.linear_streamed(x, mx["w_qkv"], scale_from=scale)
            out = torch.empty((T, self.num_heads * self.head_dim), dtype=torch.bfloat16, device=resid.device)
            ops.attention(qkv, qkv.shape[1], view.pages, ctx, view.group, out, self.num_heads, self.num_kv_heads, self.head_dim,
                          view.page_size, view.num_pages, self.window, self.scale,
                          rope=(mx["inv_freq"], mx["rotary_dim"], view.writes and view.pages is not None))
            xw, ss = ops.linear_streamed(out, mx["w_o"], add_into=(resid, f["norm2"]["weight"]))
            act = ops.linear_streamed(xw, ff["w_gate_up"], silu_mul=True, scale_from=(ss, self.hidden, f["norm2"]["eps"]))
            nxt = self.fusions[i + 1]["norm1"] if i + 1 < len(self.fusions) else None
            xw, ss = ops.linear_streamed(act, ff["w_down"], add_into=(resid, nxt["weight"] if nxt else None))
            x, scale = xw, ((ss, self.hidden, nxt["eps"]) if nxt else None)


def plan_stacks(blocks, runs, run_owner, run_group, rt) -> Dict[int, DecodeStack]:
    """Maximal stretches of the schedule that one launch can run, by the index of their first run."""
    if not (hasattr(rt.ops, "decode_stack") or hasattr(rt.ops, "linear_streamed")) or rt.dtype != torch.bfloat16:
        return {}
    stacks: Dict[int, DecodeStack] = {}
    i = 0
    while i < len(runs):
        def describe(k):
            f = blocks[runs[k].layer].decode_fusion()
            where = run_group.get(run_owner[k])
            geo = _geometry(f) if f is not None and where is not None else None
            return (f, geo, where[0]) if geo is not None else None

        here = describe(i)
        if here is None:
            i += 1
            continue
        fusions, j = [here[0]], i + 1
        while j < len(runs):
            nxt = describe(j)
            if nxt is None or nxt[1:] != here[1:]:
                break
            fusions.append(nxt[0])
            j += 1
        stacks[i] = DecodeStack(i, fusions, here[2], rt)
        i = j
    return stacks
