"""The kernels as Python calls on torch tensors.

Every function launches hand-written CUDA from the libraries under ``kernels/``
on torch's current stream; tensors are only memory here.  There is no CPU path:
without a CUDA device the constructor raises.  Matrix products of the bfloat16
path with many rows go to cuBLAS through ``torch.mm``, as the reference sends
its linears to cuBLAS through candle (models/src/llama.rs:269-271); the gate/up
product of long prompts, with its activation, runs on the tcgen05 kernel here.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1
META_HEADER_INTS = 20
META_NUM_TOKENS, META_NUM_ENTRIES, META_NUM_ROWS, META_BT_STRIDE, META_BT_OFFSET = 0, 1, 2, 4, 12
MAX_GROUPS = 8
STATUS_WORDS = 8
SKINNY_MAX_ROWS = 16  # bfloat16 linears with at most this many rows stream the weights

CORE_SOURCES = ["kernels/core.cu", "kernels/linear_bf16.cu", "kernels/linear_stream.cu", "kernels/sampling.cu"]
ATTENTION_SOURCES = ["kernels/attention_bf16.cu"]
GEMM_SOURCES = ["kernels/gemm_tcgen05.cu"]
ATTENTION_TC_SOURCES = ["kernels/attention_tcgen05.cu"]
DECODE_STACK_SOURCES = ["kernels/decode_stack.cu"]
ATTENTION_TC_HEAD_DIMS = (64, 128)  # head sizes of the tcgen05 prefill attention
ATTENTION_HEAD_DIMS = tuple(range(16, 257, 16))  # every head size the kernels take; the build check builds them all, a model only its own


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


class CudaOps:
    """Loads (building at first use) the kernel library and exposes its entry points."""

    def __init__(self, device: torch.device):
        if not torch.cuda.is_available():
            raise KernelError("this engine runs on a CUDA device only; none is available")
        self.device = torch.device(device)
        self.lib = build.load_library("core", CORE_SOURCES, cuda=True)
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=self.device)
        self.launches = 0  # own kernel launches, counted for the benchmark record
        self._attn_libs = {}
        self._attn_tc_libs = {}
        # levers for the kernel tests (each kernel is compared with the one it stands in for)
        self.tc_attention = True    # tcgen05 prefill attention where the geometry allows
        self.decode_cluster = True  # split merge of the decode attention inside a cluster
        self.tc_gemm = True         # gate/up + SwiGLU of long prompts on tcgen05
        # large decode batches: key tiles dealt out evenly over as many blocks as the GPU holds ("0": never;
        # a number above 1: always, with that many blocks, for experiments and tests)
        flat = os.environ.get("ATOMA_INFER_DECODE_FLAT", "1")
        self.decode_flat = flat != "0"
        self.decode_flat_forced = int(flat) if flat.isdigit() and int(flat) > 1 else 0
        self._flat_blocks = {}
        self._gemm_lib = None
        self.last_tokens = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)  # by state slot
        self._counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)  # split arrivals; kernels leave zeros
        # Programmatic dependent launch lets a kernel start while its predecessor drains (its weight
        # loads are in flight before the dependency wait).  Blocks that have started early wait for the
        # kernel before them and slow it down while they do, so only kernels whose wait is short start
        # early: the few-row linears and the decode attention release their dependents when they start
        # themselves; the norm kernel, which also starts early, releases its dependents only once its own
        # wait is over (else the linear after it would wait through the whole linear before it).  Measured
        # on the decode step of Llama 3.2 1B: off 0.967 ms; linears and attention 0.918 ms; with the norm
        # 0.906 ms; every kernel, each releasing its dependents at once, 1.17 ms.
        # ATOMA_INFER_PDL: "0" off, "1" every kernel, "linear" without the norm, default "linear+norm".
        mode = os.environ.get("ATOMA_INFER_PDL", "linear+norm")
        self.pdl = {"0": 0, "1": 1, "linear": 2, "linear+norm": 6}.get(mode, 6)
        self.fused_rope = True  # the decode attention rotates q and k and writes the new key and value itself
        # Few-row linears go to the persistent, TMA-fed kernel (kernels/linear_stream.cu) where it is the faster one
        # (see _stream_linear); ATOMA_INFER_STREAM_LINEAR=0 keeps them all on the kernel that loads weights into
        # fragments directly (kernels/linear_bf16.cu).  The kernel tests set the attribute.
        self.stream_linear = os.environ.get("ATOMA_INFER_STREAM_LINEAR", "1") != "0"
        self.stream_min_rows = int(os.environ.get("ATOMA_INFER_STREAM_MIN_ROWS", "1"))  # a test and measurement lever
        # In decode steps whose linears are streamed, the RMSNorms between them are folded into them (parts/decode_stack.py,
        # the chain); ATOMA_INFER_FOLD_NORMS=0 leaves the norm a kernel of its own.
        self.fold_norms = os.environ.get("ATOMA_INFER_FOLD_NORMS", "1") != "0"
        # Decode steps of at most 16 rows can run stretches of whole layers as one persistent kernel (ATOMA_INFER_FUSED_LAYERS=1;
        # off by default while it is slower than the step part by part)
        self.fused_layers = os.environ.get("ATOMA_INFER_FUSED_LAYERS", "0") == "1"
        self._stack_libs, self._stack_blocks = {}, {}
        # Before the decode attention of a small batch the weight of the linear after it is asked into L2 if it has
        # at most this many bytes (0: never); see _prefetch_next_weight.
        self.prefetch_bytes = int(float(os.environ.get("ATOMA_INFER_PREFETCH_MB", "12")) * (1 << 20))
        self._order, self._order_index, self._starts, self._cursor = [], {}, [], 0
        # ... on a stream of its own when the step has at most this many rows, else as a link of the step's chain
        self.prefetch_aside_rows = int(os.environ.get("ATOMA_INFER_PREFETCH_ASIDE_ROWS", "4"))
        self._side_stream, self._side_pending = None, False
        self.lib.kernels_set_pdl(int(self.pdl))
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, err: int, what: str):
        self.launches += 1
        if err:
            raise KernelError(f"{what}: CUDA error {err}")

    def set_pdl(self, on: bool) -> None:
        self.pdl = int(on)
        self.lib.kernels_set_pdl(int(on))
        for lib in self._attn_libs.values():
            lib.kernels_set_pdl(1 if on else 0)

    @staticmethod
    def describe_status(words) -> Optional[str]:
        """What the status words say (None: nothing).  Kernels write them instead of trapping or hanging."""
        s = list(words)
        if not any(s):
            return None
        return (f"token id out of range at token {s[0] - 1}" if s[0] else
                f"block table names no valid page for token {s[1] - 1}" if s[1] else
                f"a tensor-core GEMM block ({s[2] - 1}) gave up waiting on a barrier" if s[2] else
                f"a tensor-core attention block ({s[3] - 1}) gave up waiting on a barrier" if s[3] else
                f"a block ({s[4] - 1}) of the decode step's layer kernel gave up waiting" if s[4] else
                f"a block ({s[5] - 1}) of the streamed few-row linear gave up waiting" if s[5] else
                f"status words {s}")

    def clear_status(self) -> None:
        self.status.zero_()

    def check_status(self) -> None:
        """Raises if a kernel of an earlier launch met a bad token id or page id, or gave up a wait
        (synchronises)."""
        what = self.describe_status(self.status.tolist())
        if what:
            self.clear_status()
            raise KernelError("device status: " + what)

    # ------------------------------------------------------------------ weights ahead of time
    def set_weight_order(self, weights) -> None:
        """The weight matrices of the model's linears in the order a step streams them (a model tells this once,
        after binding)."""
        self._order = [(w.data_ptr(), w.numel() * w.element_size()) for w in weights]
        self._starts, at = [], 0
        for _, n in self._order:
            self._starts.append(at)
            at += n
        self._order_index = {}
        for i, (ptr, _) in enumerate(self._order):
            self._order_index.setdefault(ptr, []).append(i)
        self._cursor = 0

    def _note_weight(self, w) -> None:
        where = self._order_index.get(w.data_ptr())
        if where:
            self._cursor = next((k for k in where if k >= self._cursor), where[0]) + 1

    def _prefetch_next_weight(self, rows: int = 0) -> None:
        """Before the decode attention of a small batch: asks the weight of the linear after it (the next one in the
        stream after the last linear that ran) into L2, if it is a small one (``prefetch_bytes`` at most).  A small
        matrix is read in a few microseconds that are mostly start-up and drain; read from L2 it is shorter, and the
        attention of a small batch leaves the bandwidth to bring it there.  Measured, decode step at batch 8: Llama
        3.2 1B (8.4 MB) 0.924 -> 0.897 ms; asking for more than that one weight, or from inside the linears, is
        slower; at the 3B and 8B sizes (18.9 and 33.5 MB) asking at all is 3 to 5 % slower, hence the limit.
        ``rows``: the step's rows.  With at most ``prefetch_aside_rows`` of them (ATOMA_INFER_PREFETCH_ASIDE_ROWS) the
        request runs on a stream of its own beside the step's chain; measured in the chain against beside it, decode
        step of Llama 3.2 1B: batch 1 0.744 / 0.730 ms, batch 2 0.763 / 0.744, batch 4 0.773 / 0.745, batch 8 0.820 /
        0.839."""
        if self._cursor >= len(self._order):
            return
        ptr, size = self._order[self._cursor]
        if size > self.prefetch_bytes:
            return
        if rows > self.prefetch_aside_rows:
            self._check(self.lib.l2_prefetch(1, (ctypes.c_void_p * 1)(ptr), (ctypes.c_ulonglong * 1)(size), self._stream()),
                        "l2_prefetch")
            return
        # on a stream of its own, after what the step has launched so far: the attention then follows the projection
        # directly in the chain of dependent launches
        main = torch.cuda.current_stream(self.device)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(self.device)
        fork = torch.cuda.Event()
        fork.record(main)
        self._side_stream.wait_event(fork)
        self._check(self.lib.l2_prefetch_aside(1, (ctypes.c_void_p * 1)(ptr), (ctypes.c_ulonglong * 1)(size),
                                               ctypes.c_void_p(self._side_stream.cuda_stream)), "l2_prefetch")
        self._side_pending = True

    def join_side_work(self) -> None:
        """What ran beside the step's stream (see _prefetch_next_weight) joins it: called at the end of a forward pass."""
        if self._side_pending:
            done = torch.cuda.Event()
            done.record(self._side_stream)
            torch.cuda.current_stream(self.device).wait_event(done)
            self._side_pending = False

    # ------------------------------------------------------------------ kernels
    def embed(self, tokens, table, resid, meta, T: int, scale: float = 1.0):
        """resid[t] = scale * table[tokens[t]].  A token id -1 - s means: the token last sampled into slot s
        (``self.last_tokens``)."""
        H, V = table.shape[1], table.shape[0]
        self._check(self.lib.embed_rows(_p(tokens), _p(table), _code(table), _p(resid), _p(meta), T, H, V,
                                        ctypes.c_float(scale), _p(self.last_tokens), self.last_tokens.numel(),
                                        _p(self.status), self._stream()), "embed_rows")

    def add_rmsnorm(self, resid, delta, w, eps: float, out, meta, n: int, rows=None):
        """resid += delta (if given); out = rmsnorm(resid) * w.  With ``rows`` the sum and the
        norm are taken at those rows only and resid is left as it is."""
        H = resid.shape[-1]
        self._check(self.lib.add_rmsnorm(_p(resid), _p(delta), _code(delta) if delta is not None else _code(out),
                                         _p(rows), _p(w), ctypes.c_float(eps), _p(out), _code(out), _p(meta), n, H,
                                         self._stream()), "add_rmsnorm")

    def linear(self, x, w, *, out_dtype=None, silu_mul: bool = False, meta=None, use_rows: bool = False):
        """x [M, K] times w [N, K] transposed.  ``silu_mul``: w is [gate; up] stacked and the
        result is silu(gate part) * (up part), of N/2 columns."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        n_out = N // 2 if silu_mul else N
        if x.dtype == torch.float32:
            y = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._check(self.lib.gemm_f32(_p(x), _p(w), _p(y), M, N, K, self._stream()), "gemm_f32")
            if silu_mul:
                out = torch.empty((M, n_out), dtype=torch.float32, device=x.device)
                self.silu_mul(y, out, meta, M, n_out)
                return out
            return y
        if self._stream_linear(M, N, K) and x.is_contiguous() and w.is_contiguous():
            return self.linear_streamed(x, w, out_dtype=out_dtype, silu_mul=silu_mul)
        if M <= SKINNY_MAX_ROWS and K % 8 == 0:
            y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
            self._note_weight(w)
            self._check(self.lib.linear_skinny(_p(x), _p(w), _p(y), _code(y), int(silu_mul), _p(meta), int(use_rows),
                                               M, N, K, self._stream()), "linear_skinny")
            return y
        if silu_mul and out_dtype == x.dtype and self._swiglu_on_tcgen05(M, n_out, K):
            return self.gemm_tc(x, w, silu_mul=True, bn=256)
        if out_dtype == torch.float32:
            y = torch.mm(x, w.t(), out_dtype=torch.float32)
        else:
            y = torch.mm(x, w.t())
        if silu_mul:
            out = torch.empty((M, n_out), dtype=x.dtype, device=x.device)
            self.silu_mul(y, out, meta, M, n_out)
            return out
        return y

    def linear_streamed(self, x, w, *, out_dtype=None, silu_mul: bool = False, scale_from=None, add_into=None):
        """``linear`` on the TMA-fed persistent kernel whatever the policy says (bfloat16, at most 16 rows, K a multiple
        of 64, contiguous operands).  An RMSNorm can be folded into the linears around it:
        ``add_into=(resid, next_w)``: the linear before a norm.  Nothing is returned as y; the product is added into the
        float32 residual and, with ``next_w`` (the norm's weight; None if no norm follows), the call returns
        ``(xw, ss)``: the new residual times that weight in bfloat16, and per 16-column tile and row the sum of squares.
        ``scale_from=(ss, width, eps)``: the linear after the norm, given ``xw`` as x: its rows are scaled by 1 / rms."""
        M, K = x.shape
        N = w.shape[0]
        self._note_weight(w)
        ss_in, parts, width, eps = (None, 0, 0, 0.0) if scale_from is None else (scale_from[0], scale_from[0].numel() // 16,
                                                                                 scale_from[1], scale_from[2])
        if add_into is not None:
            resid, next_w = add_into
            xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if next_w is not None else None
            ss = torch.empty(-(-N // 16) * 16, dtype=torch.float32, device=x.device) if next_w is not None else None
            self._check(self.lib.linear_stream_norm(_p(x), _p(w), None, DT_BF16, 2, M, N, K, _p(ss_in), parts, width,
                                                    ctypes.c_float(eps), _p(resid), _p(next_w), _p(xw), _p(ss), _p(self.status),
                                                    self._stream()), "linear_stream_norm")
            return xw, ss
        y = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype or x.dtype, device=x.device)
        self._check(self.lib.linear_stream_norm(_p(x), _p(w), _p(y), _code(y), int(silu_mul), M, N, K, _p(ss_in), parts, width,
                                                ctypes.c_float(eps), None, None, None, None, _p(self.status), self._stream()),
                    "linear_stream_norm")
        return y

    def _stream_linear(self, M: int, N: int, K: int) -> bool:
        """Whether a bfloat16 linear of M <= 16 rows runs on the TMA-fed persistent kernel: whenever it can (K a multiple
        of 64).  Measured, decode step as a CUDA graph, all linears direct against all streamed: Llama 3.2 1B sizes, batch
        1 / 2 / 4 / 8 / 12 / 16: 0.758 / 0.800 / 0.831 / 0.878 / 1.125 / 1.265 ms against 0.778 / 0.791 / 0.805 / 0.829 /
        0.918 / 0.944, and with the norms folded into the streamed linears (up to 8 rows) 0.746 / 0.763 / - / 0.826;
        8 layers of the 3B sizes, batch 1 / 8: 0.539 / 0.656 against 0.535 (folded) / 0.641; of the 8B sizes: 0.918 / 1.040
        against 0.802 / 0.912.  The direct kernel is a quarter to a third slower with two n-tiles (9 to 16 rows).  Mixing
        the two within a layer is the slowest choice (3B sizes, batch 8: streamed only where its tiles fill the blocks
        evenly 0.733 to 0.751 ms; 1B sizes, batch 1, gate/up alone streamed 0.837): a persistent kernel holds every
        multiprocessor's shared memory until its blocks leave, so a kernel of another kind after it cannot start early.
        ``stream_min_rows`` (ATOMA_INFER_STREAM_MIN_ROWS) keeps steps of fewer rows on the direct kernel."""
        if not self.stream_linear or M > SKINNY_MAX_ROWS or K % 64:
            return False
        return M >= self.stream_min_rows

    def _swiglu_on_tcgen05(self, M: int, n_out: int, K: int) -> bool:
        """Whether the gate/up product with the SwiGLU epilogue runs on the persistent tcgen05 kernel instead
        of the library product followed by the activation kernel.  It wins when its 128 x 128 output tiles
        fill whole rounds of the multiprocessors (measured at hidden 2048, intermediate 8192: 104 against
        112 us at 2,048 rows, 198 against 213 us at 4,096; a tie at 1,536; slower below and at 3,000)."""
        if not self.tc_gemm or M < 1536 or K % 8 or n_out % 8:
            return False
        tiles = -(-M // 128) * -(-n_out // 128)
        rounds = -(-tiles // self.num_sms)
        return tiles >= 0.97 * rounds * self.num_sms

    def gemm_tc(self, a, b, *, out_dtype=None, silu_mul: bool = False, transpose: bool = False, bn: int = 256,
                ksplit: int = 1, persistent: bool = True, out=None):
        """C = A * B^T on tcgen05/TMEM with TMA-fed tiles (kernels/gemm_tcgen05.cu).  a [RA, K] fills the
        128-row side of the MMA, b [RB, K] the BN-column side.  ``transpose``: the result is [RB, RA]
        (used with a = weights when the activations have few rows).  ``silu_mul``: b is [gate; up]
        stacked and the result has RB/2 columns.  ``ksplit``: blocks of a cluster that share a tile's K.
        ``persistent`` (untransposed, unsplit): one block per multiprocessor walks the tiles and stores a tile
        while the tensor core computes the next."""
        if self._gemm_lib is None:
            self._gemm_lib = build.load_library("gemm_tcgen05", GEMM_SOURCES, cuda=True)
        out_dtype = out_dtype or a.dtype
        ra, K = a.shape
        rb = b.shape[0] // 2 if silu_mul else b.shape[0]
        shape = (rb, ra) if transpose else (ra, rb)
        c = out if out is not None else torch.empty(shape, dtype=out_dtype, device=a.device)
        self._check(self._gemm_lib.gemm_tcgen05(_p(a), _p(b), _p(c), ra, rb, K, shape[1], _code(c), int(silu_mul),
                                                int(transpose), bn, ksplit, int(persistent and not transpose and ksplit == 1),
                                                _p(self.status), self._stream()),
                    "gemm_tcgen05")
        return c

    def silu_mul(self, gu, out, meta, T: int, inter: int):
        self._check(self.lib.silu_mul(_p(gu), _p(out), _code(gu), _p(meta), T, inter, self._stream()), "silu_mul")

    def rope_kv_store(self, qkv, positions, token_entry, meta, group: int, inv_freq, cache_layer, num_pages: int,
                      T: int, nq: int, nkv: int, d: int, rot: int, page_size: int, store_kv: bool):
        self._check(self.lib.rope_kv_store(_p(qkv), _code(qkv), _p(positions), _p(token_entry), _p(meta), group,
                                           _p(inv_freq), _p(cache_layer), num_pages, T, nq, nkv, d, rot, page_size,
                                           int(store_kv), _p(self.status), self._stream()), "rope_kv_store")

    def fast_attention(self, dtype, d: int, nq: int, nkv: int, q_stride: int) -> bool:
        """Whether the tensor-core attention kernels take this geometry."""
        return (dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and nq % nkv == 0 and nq // nkv <= 16
                and q_stride % 8 == 0)

    def attention(self, q, q_stride: int, cache_layer, ctx, group: int, out, nq: int, nkv: int, d: int,
                  page_size: int, num_pages: int, window: int, scale: float, rope=None):
        """Attention of the step's queries over what their requests have cached (the step's own
        keys included).  bfloat16 with a head size in steps of 16 up to 256 runs the tensor-core
        kernels (one library per head size, built at first use); anything else, and all of
        float32, runs the plain kernel.  ``rope`` = (inv_freq, rotary_dim, store_kv): only for decode
        steps on the fast path (see ``fast_attention``); the queries are then still unrotated and the
        kernel rotates them, and writes the new key and value, itself."""
        T, S = ctx.T, ctx.S
        if rope is not None and not (ctx.decode_only and self.fast_attention(q.dtype, d, nq, nkv, q_stride)):
            raise KernelError("fused rotation exists for decode steps on the bfloat16 fast path only")
        if self.fast_attention(q.dtype, d, nq, nkv, q_stride):
            lib = self._attention_library(d)
            if ctx.decode_only:
                inv_freq, rot, store = rope if rope is not None else (None, 0, False)
                flat_blocks = self._decode_flat_blocks(lib, d, S, nkv)
                if flat_blocks:
                    # large batch: as many blocks as the GPU holds share all key tiles evenly
                    n = lib.attn_decode_flat_scratch_floats(S, nq, nkv, flat_blocks)
                    scratch = torch.empty(n, dtype=torch.float32, device=q.device)
                    if S * nkv > self._counters.numel():
                        raise KernelError(f"decode attention: {S} requests x {nkv} heads exceed the split counters")
                    self._check(lib.attn_decode_flat(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group,
                                                     _p(ctx.cu_tokens), _p(ctx.positions), _p(out), _p(scratch),
                                                     _p(self._counters), _p(inv_freq), rot, int(store), S, nq, nkv,
                                                     page_size, num_pages, window, ctypes.c_float(scale), flat_blocks,
                                                     _p(self.status), self._stream()), "attn_decode_flat")
                    return
                splits = self.decode_splits(S, nkv, ctx.max_context, lib.attn_decode_blocks_per_sm())
                # the splits merge inside a thread-block cluster when they fit one, else through scratch
                if S <= SKINNY_MAX_ROWS:
                    self._prefetch_next_weight(S)
                cluster = self.decode_cluster and 1 < splits <= lib.attn_decode_max_cluster()
                n = 0 if cluster else lib.attn_decode_scratch_floats(S, nq, splits)
                scratch = torch.empty(n, dtype=torch.float32, device=q.device) if n else None
                if not cluster and S * nkv > self._counters.numel():
                    raise KernelError(f"decode attention: {S} requests x {nkv} heads exceed the split counters")
                self._check(lib.attn_decode(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                            _p(ctx.positions), _p(out), _p(scratch), _p(self._counters), _p(inv_freq),
                                            rot, int(store), S, nq, nkv, page_size, num_pages,
                                            window, ctypes.c_float(scale), splits, int(cluster), ctx.max_context,
                                            _p(self.status), self._stream()),
                            "attn_decode")
            elif self._prefill_tc(d, page_size, nq, nkv) is not None:
                tc = self._prefill_tc(d, page_size, nq, nkv)
                self._check(tc.attn_prefill_tc(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                               _p(ctx.context_lens), _p(out), S, ctx.max_tokens_per_entry, nq, nkv,
                                               page_size, num_pages, window, ctypes.c_float(scale), ctx.max_context,
                                               _p(self.status), self._stream()), "attn_prefill_tc")
            else:
                self._check(lib.attn_prefill(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                             _p(ctx.context_lens), _p(out), S, ctx.max_tokens_per_entry, nq, nkv,
                                             page_size, num_pages, window, ctypes.c_float(scale), ctx.max_context,
                                             _p(self.status), self._stream()), "attn_prefill")
            return
        if d > 256:
            raise KernelError(f"head size {d} is not supported (at most 256)")
        self._check(self.lib.attn_generic(_p(q), q_stride, _p(cache_layer), _code(q), _p(ctx.meta), group,
                                          _p(ctx.token_entry), _p(ctx.positions), _p(out), T, nq, nkv, d, page_size,
                                          num_pages, window, ctypes.c_float(scale), _p(self.status), self._stream()),
                    "attn_generic")

    # ------------------------------------------------------------------ whole layers of a decode step
    def _decode_stack_library(self, d: int):
        lib = self._stack_libs.get(d)
        if lib is None:
            lib = build.load_library(f"decode_stack_d{d}", DECODE_STACK_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            lib.decode_stack_scratch_floats.restype = ctypes.c_size_t
            if lib.decode_stack_head_dim() != d:
                raise KernelError(f"decode stack library was built for head size {lib.decode_stack_head_dim()}, wanted {d}")
            self._stack_libs[d] = lib
        return lib

    def decode_stack_layers(self, layers, *, d: int, hidden: int, intermediate: int, nq: int, nkv: int, page_size: int,
                            num_pages: int) -> torch.Tensor:
        """The layer kernel's descriptors on the device, one per dict of ``layers`` (tensors ``w_qkv``, ``w_o``,
        ``w_gate_up``, ``w_down``, ``norm1``, ``norm2``, ``inv_freq``, ``cache``; bool ``store_kv``)."""
        lib = self._decode_stack_library(d)
        size = int(lib.decode_stack_layer_bytes())
        host = torch.zeros(len(layers) * size, dtype=torch.uint8)
        for i, ly in enumerate(layers):
            err = lib.decode_stack_fill_layer(ctypes.c_void_p(host.data_ptr() + i * size), _p(ly["w_qkv"]), _p(ly["w_o"]),
                                              _p(ly["w_gate_up"]), _p(ly["w_down"]), _p(ly["norm1"]), _p(ly["norm2"]),
                                              _p(ly["inv_freq"]), _p(ly["cache"]), int(ly["store_kv"]), hidden, intermediate,
                                              nq, nkv, page_size, num_pages)
            if err:
                raise KernelError(f"decode_stack_fill_layer: error {err} (widths must be multiples of 64)")
        return host.to(self.device)

    def decode_stack_record_clocks(self, d: int, buffer: Optional[torch.Tensor]) -> None:
        """For measurements: the next launches of the layer kernel leave the global clock after every phase and every
        barrier of every layer in ``buffer`` (int64 [blocks, layers, 10]; None: off).  Reading that clock costs each
        block a few hundred nanoseconds a time."""
        self._decode_stack_library(d).decode_stack_set_times(_p(buffer))

    def decode_stack_blocks(self, d: int, rows: int, hidden: int) -> int:
        """Blocks the layer kernel would run with for ``rows`` rows of width ``hidden`` (the larger of the model's
        width and heads x head size; 0: it does not take them)."""
        key = (d, rows <= 8, hidden)
        n = self._stack_blocks.get(key)
        if n is None:
            ok = d % 16 == 0 and 16 <= d <= 256 and hidden % 8 == 0
            n = self._stack_blocks[key] = int(self._decode_stack_library(d).decode_stack_blocks(rows, hidden)) if ok else 0
        return n if rows <= SKINNY_MAX_ROWS else 0

    def decode_stack(self, layers, num_layers: int, resid, delta, arrivals, ctx, group: int, *, hidden: int, intermediate: int,
                     nq: int, nkv: int, d: int, rot: int, window: int, page_size: int, num_pages: int, eps: float,
                     scale: float, all_store_kv: bool = True):
        """``num_layers`` pre-norm layers (RMSNorm, rotary attention over the paged cache, SwiGLU) of a decode step in
        one launch (kernels/decode_stack.cu): resid [rows, hidden] float32 is updated in place, ``delta`` added first."""
        lib = self._decode_stack_library(d)
        M = ctx.T
        blocks = self.decode_stack_blocks(d, M, max(hidden, nq * d))
        if not blocks or ctx.S != M or not ctx.decode_only:
            raise KernelError("the decode layer kernel takes decode steps of at most 16 rows")
        if M * nkv > self._counters.numel():
            raise KernelError(f"decode layers: {M} requests x {nkv} heads exceed the split counters")
        dev = resid.device
        qkv = torch.empty((M, (nq + 2 * nkv) * d), dtype=torch.bfloat16, device=dev)
        out = torch.empty((M, nq * d), dtype=torch.bfloat16, device=dev)
        act = torch.empty((M, intermediate), dtype=torch.bfloat16, device=dev)
        xw = torch.empty((M, hidden), dtype=torch.bfloat16, device=dev)
        ss_part = torch.empty(-(-hidden // 16) * 16, dtype=torch.float32, device=dev)
        scratch = torch.empty(lib.decode_stack_scratch_floats(M, nq, nkv, blocks), dtype=torch.float32, device=dev)
        self._check(lib.decode_stack(_p(layers), num_layers, _p(resid), _p(delta), _p(qkv), _p(out), _p(act), _p(xw), _p(ss_part), _p(scratch),
                                     _p(self._counters), _p(arrivals), _p(ctx.meta), group, _p(ctx.cu_tokens), _p(ctx.positions),
                                     M, ctx.S, hidden, intermediate, nq, nkv, rot, window, page_size, num_pages,
                                     ctypes.c_float(eps), ctypes.c_float(scale), int(all_store_kv), _p(self.status), self._stream()),
                    "decode_stack")

    def _decode_flat_blocks(self, lib, d: int, S: int, nkv: int) -> int:
        """Grid size of the flat decode kernel if this batch should take it (at least half as many (request,
        head group) pairs as blocks the GPU holds: below that, fixed splits in clusters fill the GPU as well
        and merge faster), else 0."""
        if not self.decode_flat:
            return 0
        if self.decode_flat_forced:
            return self.decode_flat_forced
        key = (d, S)
        blocks = self._flat_blocks.get(key)
        if blocks is None:
            blocks = self._flat_blocks[key] = int(lib.attn_decode_flat_blocks(S))
        return blocks if blocks and 2 * S * nkv >= blocks else 0

    def _prefill_tc(self, d: int, page_size: int, nq: int, nkv: int):
        """The tcgen05 prefill attention library for this geometry, or None (then the mma.sync kernel runs)."""
        if d not in ATTENTION_TC_HEAD_DIMS or not self.tc_attention:
            return None
        lib = self._attn_tc_libs.get(d)
        if lib is None:
            lib = build.load_library(f"attention_tc_d{d}", ATTENTION_TC_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            if lib.attn_tc_head_dim() != d:
                raise KernelError(f"tcgen05 attention library was built for head size {lib.attn_tc_head_dim()}, wanted {d}")
            self._attn_tc_libs[d] = lib
        return lib if lib.attn_prefill_tc_supports(page_size, nq, nkv) else None

    def _attention_library(self, d: int):
        lib = self._attn_libs.get(d)
        if lib is None:
            lib = build.load_library(f"attention_d{d}", ATTENTION_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            lib.attn_decode_scratch_floats.restype = ctypes.c_size_t
            lib.attn_decode_flat_scratch_floats.restype = ctypes.c_size_t
            lib.kernels_set_pdl(1 if self.pdl else 0)
            if lib.attn_head_dim() != d:
                raise KernelError(f"attention library was built for head size {lib.attn_head_dim()}, wanted {d}")
            self._attn_libs[d] = lib
        return lib

    def decode_splits(self, S: int, nkv: int, max_context: int, blocks_per_sm: int = 2) -> int:
        """Splits of the key range per (request, key/value head) in a decode step.  Few requests:
        as many splits as keep all blocks resident at once, at most 8 (one cluster, which merges through its
        shared memory) and at least 256 keys each; a long context of very few requests takes more than 8 (at
        least 512 keys each, merged through scratch by the last block to arrive) when that at least doubles the
        blocks (one request of 32,768 keys: 43 -> 25 us a layer).  Many requests (more blocks than fit at
        once): the smallest count up to 4 whose last wave is at least 85 % as full as the best
        (the reference's heuristic has this shape, csrc/src/lib.rs:2122-2199)."""
        blocks = max(S * nkv, 1)
        capacity = self.num_sms * max(blocks_per_sm, 1)
        most = max(1, max_context // 256)
        if blocks < capacity:
            few = max(1, min(8, most, capacity // blocks))
            many = min(capacity // blocks, max_context // 512)
            return many if many >= 2 * few else few

        def efficiency(s):
            waves = blocks * s / capacity
            return waves / -(-blocks * s // capacity)

        most = min(most, 4)
        best = max(efficiency(s) for s in range(1, most + 1))
        return next(s for s in range(1, most + 1) if efficiency(s) >= 0.85 * best)

    def sample(self, logits, temperature, top_k, top_p, seed, step, out, num_rows=None, slots=None):
        """``slots`` (int32 per row): also leave each token in ``self.last_tokens[slot]`` for the next step."""
        R, V = logits.shape
        self._check(self.lib.sample_rows(_p(logits), R, V, _p(temperature), _p(top_k), _p(top_p), _p(seed), _p(step),
                                         _p(out), _p(num_rows), _p(slots), _p(self.last_tokens), self._stream()),
                    "sample_rows")

    def repeat_penalty(self, row, penalty: float, context):
        self._check(self.lib.repeat_penalty(_p(row), row.numel(), ctypes.c_float(penalty), _p(context),
                                            context.numel(), self._stream()), "repeat_penalty")
