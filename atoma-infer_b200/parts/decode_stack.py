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


def plan_stacks(blocks, runs, run_owner, run_group, rt) -> Dict[int, DecodeStack]:
    """Maximal stretches of the schedule that one launch can run, by the index of their first run."""
    if not hasattr(rt.ops, "decode_stack") or rt.dtype != torch.bfloat16:
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
