"""The call table of the CUDA extension: torch tensors in, kernels launched on torch's current stream.

Every function here launches hand-written sm_100a kernels from this folder's
``.cu`` files through their ``extern "C"`` entry points.  Matrix products in
bfloat16 with many rows go to cuBLAS through ``torch.matmul``, where the
reference's engine calls the same library (engine/model.py:291,295,297,299).
There is no CPU path and no other backend: without a CUDA device or without
the compiled library, ``get_ops`` raises.
"""

from __future__ import annotations

import contextlib
import ctypes
import weakref
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .build import BuildError, load

F32, BF16 = 0, 1
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # (device index) -> cudaStream_t as an int


class KernelError(RuntimeError):
    """A kernel launch was refused (sizes it does not take) or failed."""


class SbBatch(Structure):
    _fields_ = [("seq_slot", c_void_p), ("cu_q", c_void_p), ("row_seq", c_void_p), ("lengths", c_void_p),
                ("n_seqs", c_int), ("n_rows", c_int), ("null_slot", c_int), ("reserved", c_int)]


class SbKV(Structure):
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("table", c_void_p), ("table_width", c_int),
                ("ring_pages", c_int), ("n_kv_heads", c_int), ("head_dim", c_int)]


class SbFusedQK(Structure):
    _fields_ = [("qkv", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
                ("status", c_void_p), ("eps", c_float), ("norm_f32", c_int), ("store_kv", c_int), ("reserved", c_int),
                ("next_w", c_void_p), ("next_bytes", c_longlong)]


class SbFlex(Structure):
    _fields_ = [("q", c_void_p), ("q_row", c_longlong), ("q_head", c_longlong), ("k", c_void_p), ("v", c_void_p),
                ("table", c_void_p), ("head_scale", c_void_p), ("slopes", c_void_p), ("sink", c_void_p),
                ("table_width", c_int), ("ring_pages", c_int), ("n_heads", c_int), ("n_kv_heads", c_int), ("k_dim", c_int),
                ("v_dim", c_int), ("v_row", c_int), ("window", c_int), ("chunk", c_int), ("scale", c_float), ("v_heads", c_int),
                ("pinned_pages", c_int), ("keep_first", c_int), ("softcap", c_float), ("talk", c_void_p)]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


class Ops:
    name = "cuda"

    # bfloat16 products with at most this many rows stay on this library's own kernels
    GENERAL_GEMM_MAX_WORK = 1 << 22

    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        self.launches = 0  # kernels of this library launched so far (cuBLAS calls are not counted)
        lib.sb_error_string.restype = ctypes.c_char_p
        lib.sb_tile_matrix_elements.restype = c_longlong
        lib.sb_tile_matrix_elements.argtypes = [c_int, c_int, c_int]
        lib.sb_error_string.argtypes = [c_int]
        sig = {
            "sb_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_gather_rows": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "sb_rmsnorm": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
            "sb_swiglu": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "sb_advance_lengths": [SbBatch, c_void_p, c_void_p],
            "sb_gemm_general": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "sb_qk_rope_store": [c_int, c_int, c_void_p, c_void_p, SbBatch, SbKV, c_int, c_int, c_void_p, c_void_p,
                                 c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
            "sb_attention_general": [c_int, c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_void_p],
            "sb_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p, c_void_p, c_void_p, c_void_p],
            "sb_gemm_skinny_gated": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                     c_void_p, c_void_p, c_void_p],
            "sb_gemm_skinny_xielu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                     c_void_p, c_void_p, c_void_p],
            "sb_gemm_skinny_normed": [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
            "sb_tile_matrix": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "sb_gemm_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p],
            "sb_gemm_stream_plan": [c_int, c_int, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)],
            "sb_attn_prefill_tc": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_attn_prefill": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p],
            "sb_attn_decode_balanced": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p],
            "sb_attn_decode": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
            "sb_attn_decode_balanced_fused": [SbFusedQK, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p,
                                              c_void_p, c_void_p],
            "sb_attn_decode_fused": [SbFusedQK, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p],
            "sb_embed_wide": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_grouped_rmsnorm": [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_float, c_void_p],
            "sb_gated_clamp": [c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p],
            "sb_tanh": [c_int, c_void_p, c_void_p, c_longlong, c_void_p],
            "sb_gemm_heads": [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_int,
                              c_int, c_int, c_void_p],
            "sb_flex_attention_general": [c_int, SbFlex, SbBatch, c_void_p, c_void_p],
            "sb_flex_attention_mma": [SbFlex, SbBatch, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
            "sb_flex_attention_rows64": [SbFlex, SbBatch, c_void_p, c_int, c_int, c_void_p],
            "sb_kv_store": [c_int, c_void_p, c_longlong, c_void_p, c_longlong, SbBatch, SbFlex, c_int, c_float, c_void_p, c_void_p],
            "sb_rotate_pairs": [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, SbBatch, c_void_p,
                                c_int, c_int, c_int, c_void_p],
            "sb_latent_prepare": [c_int, c_int, c_void_p, c_void_p, SbBatch, SbFlex, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
            "sb_token_shift": [c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, SbBatch, c_int, c_void_p,
                               c_void_p],
            "sb_wkv_scan": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                            c_void_p, c_int, c_void_p, c_longlong, c_int, SbBatch, c_int, c_int, c_void_p, c_void_p],
            "sb_embed_streams": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
            "sb_stream_norm": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                               c_int, c_float, c_void_p],
            "sb_rotate_half_store": [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, SbBatch,
                                     SbFlex, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p],
            "sb_diff_combine": [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_longlong,
                                c_void_p],
            "sb_mlstm_scan": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p,
                              c_void_p, c_float, c_void_p, c_float, c_float, c_float, c_void_p, c_longlong, SbBatch, c_int, c_int, c_int,
                              c_void_p, c_longlong, c_void_p, c_void_p],
            "sb_conv_qk_store": [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_float, c_int, c_void_p, SbBatch, SbFlex, c_int,
                                 c_void_p, c_void_p],
            "sb_head_gate": [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_void_p],
            "sb_add_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p],
            "sb_add_bias": [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p],
            "sb_scaled_sum": [c_int, c_void_p, c_float, c_void_p, c_float, c_void_p, c_longlong, c_void_p],
            "sb_relu2": [c_int, c_void_p, c_void_p, c_longlong, c_void_p],
            "sb_gemm_skinny_relu2": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p],
            "sb_gla_scan": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float,
                            c_float, c_float, c_void_p, c_longlong, SbBatch, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
            "sb_moe_route": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_float, c_void_p],
            "sb_moe_sort": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
            "sb_moe_gather": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_moe_pairs": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_float, c_int, c_void_p],
            "sb_moe_combine": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_void_p],
            "sb_embed_sinusoid": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, SbBatch, c_int, c_int, c_void_p, c_void_p],
            "sb_causal_conv": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, SbBatch, c_int, c_int, c_void_p, c_void_p],
            "sb_branch_norm_add": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_float,
                                   c_void_p, c_void_p],
            "sb_xielu": [c_int, c_void_p, c_void_p, c_longlong, c_float, c_float, c_void_p],
            "sb_talking_attention_general": [c_int, SbFlex, SbBatch, c_void_p, c_int, c_void_p, c_void_p],
            "sb_talking_attention_mma": [SbFlex, SbBatch, c_void_p, c_int, c_int, c_void_p, c_void_p],
            "sb_qk_norm_store": [c_int, c_void_p, c_void_p, SbBatch, SbFlex, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p],
            "sb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
            "sb_sample": [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_ulonglong, c_void_p, c_void_p, c_int,
                          c_void_p, c_void_p],
        }
        for name, argtypes in sig.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        for fn in (lib.sb_flex_attention_mma_smem, lib.sb_flex_attention_rows64_smem, lib.sb_talking_attention_mma_smem):
            fn.argtypes = [c_int, c_int, c_int, c_int]
            fn.restype = c_longlong
        lib.sb_set_pdl.argtypes = [c_int]
        lib.sb_set_pdl.restype = None
        self._scratch = {}
        self._sm_count = None
        self.force_skinny = None  # (K slices, tiled, warps) for tests and tuning runs; None = the rules below
        self._tiled_bytes = 0     # bytes of tile-major copies alive (a copy hangs on its matrix as ._sb_tiled = (copy, halves))
        self.decode_copy = os.environ.get("STARTER_B200_DECODE_COPY", "auto")   # "1", "0" or "auto"
        self.use_stream = os.environ.get("STARTER_B200_STREAM", "1") != "0"  # the TMA + tcgen05 product for decode
        self._kernel_status = None
        self._status_override = None
        self.decode_balanced = os.environ.get("STARTER_B200_ATTN", "balanced") != "split"
        self.force_decode_route = os.environ.get("STARTER_B200_ATTN_ROUTE") or None   # "split" or "balanced", for tests and tuning runs; None = the rule in _decode_route
        self.fuse_qk = os.environ.get("STARTER_B200_FUSE_QK", "1") != "0"
        # With the balanced kernel (more pairs than blocks fit at once) the preparation stays a kernel of its own: a block
        # walks several (sequence, kv head) pairs one after another and pays each pair's preparation on its own path.
        # Measured in the step (4B sizes, context 4,096): batch 64 8.74 ms with the preparation inside, 8.54 ms apart;
        # the split-key kernel is the other way round (batch 32: 5.41 inside, 5.53 apart).
        self.fuse_qk_balanced = os.environ.get("STARTER_B200_FUSE_QK_BALANCED", "0") != "0"
        self.prefetch_next_bytes = int(os.environ.get("STARTER_B200_PREFETCH_MAX", 24 << 20))
        self.prefill_tensor_memory = os.environ.get("STARTER_B200_PREFILL", "tc") != "mma"
        self.flex_tensor_cores = os.environ.get("STARTER_B200_FLEX", "mma") != "general"   # "general": the warp-per-row kernel only

    # ---- plumbing -----------------------------------------------------------------------

    @staticmethod
    def _stream():
        """torch's current stream as a raw handle.  Asked for at every launch: torch.cuda.current_stream() builds a
        Stream object and costs the host ~14 us a call (measured: a quarter of the host's time in an eager step);
        the raw query is a fraction of a microsecond."""
        if _RAW_STREAM is not None:
            return c_void_p(_RAW_STREAM(torch.cuda.current_device()))
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code:
            raise KernelError(f"{what}: {self.lib.sb_error_string(code).decode()} (code {code})")

    @staticmethod
    def _batch(ctx) -> SbBatch:
        b = ctx.scratch.get("sb_batch")
        if b is None:
            b = SbBatch(ctx.seq_slot.data_ptr(), ctx.cu_q.data_ptr(), ctx.row_seq.data_ptr(), ctx.lengths.data_ptr(),
                        ctx.n_seqs, ctx.n_rows, ctx.cache.null_slot, 0)
            ctx.scratch["sb_batch"] = b
        return b

    @staticmethod
    def _kv(layer_cache) -> SbKV:
        kv = getattr(layer_cache, "_sb_kv", None)
        if kv is None:
            g = layer_cache.group
            kv = SbKV(layer_cache.k.data_ptr(), layer_cache.v.data_ptr(), g.table.data_ptr(), g.table_width,
                      g.ring_pages, g.request.num_kv_heads, g.request.head_dim)
            layer_cache._sb_kv = kv
        return kv

    def set_dependent_launch(self, on: bool) -> None:
        """Launch kernels so that each may start its preamble (weight fetches, barrier set-up) while the
        one before it in the stream is finishing; see common.cuh."""
        self.lib.sb_set_pdl(int(bool(on)))

    DECODE_COPY_SHARE = 0.2   # "auto": tile-major copies are made while they stay below this share of the device's memory

    def _forget_copy(self, nbytes: int) -> None:
        self._tiled_bytes -= nbytes

    def prepare_matrix(self, w: torch.Tensor, halves: int = 1) -> torch.Tensor:
        """A weight matrix [out, in] as the products want it: contiguous, in the run's dtype.  ``halves``: 2 for
        a fused [gate; up] matrix (linear_swiglu pairs row r of the first half with row r of the second).

        For bfloat16 matrices a second, tile-major copy is kept for the decode product (gemm_skinny.cu: one
        contiguous piece per warp and turn instead of sixteen short ones; 4-7% of a decode step on the 4B
        shapes), as long as all such copies together stay below DECODE_COPY_SHARE of the device's memory
        (STARTER_B200_DECODE_COPY=1 always, =0 never).  Products with many rows read the row-major matrix."""
        if w.dim() != 2:
            raise KernelError(f"a weight matrix has two axes, got shape {tuple(w.shape)}")
        _code(w.dtype)
        w = w.contiguous()
        if (w.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[0] % halves == 0
                and self.decode_copy != "0" and getattr(w, "_sb_tiled", None) is None):
            rows = w.shape[0] // halves
            n = self.lib.sb_tile_matrix_elements(rows, w.shape[1], halves)
            total = torch.cuda.get_device_properties(w.device).total_memory
            if self.decode_copy == "1" or self._tiled_bytes + 2 * n <= self.DECODE_COPY_SHARE * total:
                tiled = torch.empty(n, dtype=torch.bfloat16, device=w.device)
                self._check(self.lib.sb_tile_matrix(_ptr(w), _ptr(tiled), rows, w.shape[1], halves, self._stream()), "tile_matrix")
                w._sb_tiled = (tiled, halves)   # lives and dies with the matrix object that the parts hold
                self._tiled_bytes += 2 * n
                weakref.finalize(w, self._forget_copy, 2 * n)
        return w

    # ---- rows ---------------------------------------------------------------------------

    def embed(self, tokens, table, status, out_float32=False):
        """Rows of the table by token id; ``out_float32``: a bfloat16 table's rows widened to 32-bit (for a model
        whose residual stream is 32-bit in every run)."""
        if out_float32 and table.dtype == torch.bfloat16:
            out = torch.empty((tokens.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
            self._check(self.lib.sb_embed_wide(_ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0], table.shape[1],
                                               table.shape[0], _ptr(status), self._stream()), "embed_wide")
            return out
        out = torch.empty((tokens.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        self._check(self.lib.sb_embed(_code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0],
                                      table.shape[1], table.shape[0], _ptr(status), self._stream()), "embed")
        return out

    def gather_rows(self, x, rows):
        out = torch.empty((rows.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
        self._check(self.lib.sb_gather_rows(_code(x.dtype), _ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1],
                                            self._stream()), "gather_rows")
        return out

    def _norm_dtypes(self, x, w):
        if x.dtype == torch.float32 and w.dtype != torch.float32:
            raise KernelError("a float32 run needs float32 norm weights")
        return _code(x.dtype), _code(w.dtype)

    def rmsnorm(self, x, w, eps):
        dt, wdt = self._norm_dtypes(x, w)
        out = torch.empty_like(x)
        self._check(self.lib.sb_rmsnorm(dt, wdt, _ptr(x), None, _ptr(w), _ptr(out), x.shape[0], x.shape[1], eps,
                                        self._stream()), "rmsnorm")
        return out

    def add_rmsnorm(self, x, delta, w, eps):
        dt, wdt = self._norm_dtypes(x, w)
        out = torch.empty_like(x)
        self._check(self.lib.sb_rmsnorm(dt, wdt, _ptr(x), _ptr(delta), _ptr(w), _ptr(out), x.shape[0], x.shape[1], eps,
                                        self._stream()), "add_rmsnorm")
        return out

    def grouped_rmsnorm(self, x, deltas, w, groups, eps, out_dtype):
        """RMSNorm of x's rows in ``groups`` equal consecutive parts, times w, in ``out_dtype``.  With ``deltas`` (one or
        two tensors of ``out_dtype``) x += their sum first, in place and in x's own type; x may be 32-bit in a
        bfloat16 run."""
        if len(deltas) > 2:
            raise KernelError("the grouped norm adds up to two branch outputs")
        if x.dtype == torch.bfloat16 and out_dtype != torch.bfloat16:
            raise KernelError("bfloat16 rows are normed into bfloat16")
        if out_dtype == torch.float32 and w.dtype != torch.float32:
            raise KernelError("a float32 run needs float32 norm weights")
        for d in deltas:
            if d.dtype != out_dtype or d.shape != x.shape or not d.is_contiguous():
                raise KernelError("a branch output has the run's dtype and the residual's shape")
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        d1 = deltas[0] if deltas else None
        d2 = deltas[1] if len(deltas) > 1 else None
        self._check(self.lib.sb_grouped_rmsnorm(_code(x.dtype), _code(out_dtype), _code(w.dtype), _ptr(x), _ptr(d1), _ptr(d2),
                                                _ptr(w), _ptr(out), x.shape[0], x.shape[1], int(groups), float(eps),
                                                self._stream()), "grouped_rmsnorm")
        return out

    def gated_clamp(self, gu, alpha, limit):
        """[g | u] -> g' * sigmoid(alpha g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)."""
        inter = gu.shape[1] // 2
        out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
        self._check(self.lib.sb_gated_clamp(_code(gu.dtype), _ptr(gu), _ptr(out), gu.shape[0], inter, float(alpha), float(limit),
                                            self._stream()), "gated_clamp")
        return out

    def tanh(self, x):
        out = torch.empty_like(x)
        self._check(self.lib.sb_tanh(_code(x.dtype), _ptr(x), _ptr(out), x.numel(), self._stream()), "tanh")
        return out

    def swiglu(self, gu):
        inter = gu.shape[1] // 2
        out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
        self._check(self.lib.sb_swiglu(_code(gu.dtype), _ptr(gu), _ptr(out), gu.shape[0], inter, self._stream()), "swiglu")
        return out

    def advance_lengths(self, ctx):
        self._check(self.lib.sb_advance_lengths(self._batch(ctx), _ptr(ctx.lengths), self._stream()), "advance_lengths")

    # ---- products -----------------------------------------------------------------------

    # The mma.sync product takes up to 32 rows.  Measured in the step (B200): to 16 rows it beats cuBLAS + the SwiGLU
    # kernel (1.7B sizes at batch 16: 1.84 -> 1.76 ms a step, 4B sizes: 3.89 -> 3.82 ms), from 17 rows on it needs 128
    # registers and loses (4B sizes at batch 32: 6.64 against 5.35 ms).
    SKINNY_MAX_ROWS = int(os.environ.get("STARTER_B200_SKINNY_MAX_ROWS", 16))
    STREAM_MIN_ROWS = 9   # the TMA + tcgen05 product serves the output head from here on
    STREAM_MAX_ROWS = 32   # 778 MB head, us by rows (this kernel / cuBLAS): 16: 126 / 132, 32: 130 / 134, 48: 137 / 131, 64: 138 / 133
    STREAM_MIN_WORK = int(os.environ.get("STARTER_B200_STREAM_MIN", 300_000_000))  # elements of W below which the simpler kernels do as well

    def kernel_status(self, device) -> torch.Tensor:
        """A status word of the kernels that are not tied to a step (bit 4: a wait inside a kernel timed out)."""
        if self._status_override is not None:
            return self._status_override
        if self._kernel_status is None:
            self._kernel_status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._kernel_status

    @contextlib.contextmanager
    def status_into(self, word: torch.Tensor):
        """While this is open, kernels that are not tied to a step raise their bits in ``word`` (int32 [1] on
        the device): a captured step then carries all its status in the word that travels with its tokens."""
        before, self._status_override = self._status_override, word
        try:
            yield
        finally:
            self._status_override = before

    def read_kernel_status(self) -> int:
        if self._kernel_status is None:
            return 0
        bits = int(self._kernel_status.item())
        if bits:
            self._kernel_status.zero_()
        return bits

    def _stream_product(self, a, w, n_out, gate_up, out_float32):
        """The TMA + tcgen05 weight-streaming product (see gemm_stream.cu)."""
        M, K = a.shape
        key = ("gemm_stream", a.device, n_out, K, gate_up, M <= 16, M <= 32)
        plan = self._scratch.get(key)
        if plan is None:
            grid, tiles, parts = c_int(), c_int(), c_int()
            self.lib.sb_gemm_stream_plan(n_out, K, self.sm_count(), ctypes.byref(grid), ctypes.byref(tiles), ctypes.byref(parts))
            bn = 16 if M <= 16 else (32 if M <= 32 else 64)
            floats = tiles.value * parts.value * bn * (2 if gate_up else 1) * 128
            plan = (grid.value, parts.value, torch.empty(floats, dtype=torch.float32, device=a.device),
                    torch.zeros(tiles.value, dtype=torch.int32, device=a.device))
            self._scratch[key] = plan
        grid, parts, partial, counters = plan
        out = torch.empty((M, n_out), dtype=torch.float32 if out_float32 else torch.bfloat16, device=a.device)
        self._check(self.lib.sb_gemm_stream(_ptr(a), _ptr(w), _ptr(out), M, n_out, K, int(gate_up), int(out_float32), grid,
                                            parts, _ptr(partial), _ptr(counters), _ptr(self.kernel_status(a.device)),
                                            self._stream()), "gemm_stream")
        return out

    def _takes_stream(self, M, n_out, K, gate_up) -> bool:
        """Measured on a B200 (microbench.py): per launch the TMA-fed kernel pays about 9 us before and
        after it streams (set-up, first data, the pass through scratch for shared tiles) and then streams
        at 6.3-6.9 TB/s; the warp-level kernel pays about 3 us and streams at 4.7 TB/s, more on very large
        matrices.  So: the output head for 9 to 32 rows, nothing smaller; from 33 rows on cuBLAS is ahead there too."""
        return (self.use_stream and self.STREAM_MIN_ROWS <= M <= (32 if gate_up else self.STREAM_MAX_ROWS)
                and K % 8 == 0 and K >= 64 and n_out * K * (2 if gate_up else 1) >= self.STREAM_MIN_WORK)

    def skinny_splits(self, blocks: int, K: int) -> int:
        """K slices per block of 16 weight rows: enough blocks for three per SM, but no slice
        shorter than 3072 columns (measured on the 4B shapes, in the decode step, with the slices
        meeting through cluster shared memory: short slices cost more in the meeting than they
        gain in parallelism; 1 slice for q/k/v, output and gate/up, 3 for down)."""
        return max(1, min(round(3 * self.sm_count() / blocks), K // 3072))

    def skinny_warps(self, n_blocks: int, nt: int = 1) -> int:
        """Warps per block.  Eight-warp blocks fit four to an SM (two from 17 rows on, where the kernel takes 128
        registers); when the blocks number a little more than that (608 for 592 places), the few left over run as a
        second wave on an empty GPU.  Four-warp blocks fit twice as many to an SM, so the same blocks run at once."""
        resident8 = (4 if nt <= 2 else 2) * self.sm_count()
        return 4 if resident8 < n_blocks <= (2 if nt <= 2 else 2.2) * resident8 else 8

    # Rows up to which a layer's norms and residual sums run inside its products (gemm_skinny.cuh) instead of in the
    # norm kernel.  Off: measured in the decode step on a B200 (4B layer sizes, context 4,096), the fold removes 72
    # of 259 launches and still loses: batch 1: 2.155 -> 2.194 ms a step, batch 8: 2.810 -> 2.889, batch 16: 3.765 ->
    # 4.301.  Every block of 16 weight rows norms all the activation rows again (608 blocks do the work of 8), and
    # that costs more than the launch it saves (about 2 us: a step without any norm is 0.12 to 0.15 ms shorter).
    FOLD_MAX_ROWS = int(os.environ.get("STARTER_B200_FOLD_MAX_ROWS", 0))

    def folds(self, rows: int, dtype) -> bool:
        """Whether a step of this many rows should hand its norms and residual sums to ``linear`` and
        ``linear_swiglu`` (``norm=``, ``add_to=``).  The decode product can take them for bfloat16, up to 16 rows
        and inner sizes that are multiples of 8."""
        return dtype == torch.bfloat16 and rows <= min(self.FOLD_MAX_ROWS, self.SKINNY_MAX_ROWS, 16)

    def _can_fold(self, rows: int, dtype, K: int) -> bool:
        return dtype == torch.bfloat16 and rows <= min(self.SKINNY_MAX_ROWS, 16) and K % 8 == 0

    def _skinny(self, a, w, n_out, gate_up, out_float32, norm=None, add_to=None, act=None, unary=None):
        """The weight-streaming product for a handful of rows (see gemm_skinny.cuh).

        norm: (weight, eps) or (weight, eps, stats) of an RMSNorm to take of a's rows first; stats is what the product
        that wrote a left behind (below), without it every block reads the rows once more.
        add_to: a bfloat16 [M, n_out] tensor that the product is added to, or an object with such a tensor as ``x``
        and a field ``stats`` (a residual stream), which then receives the statistics of the new rows: the sums of
        squares of each 16 columns, [M, ceil(n_out / 16)] floats."""
        M, K = a.shape
        blocks = -(-n_out // 16)
        want = self.skinny_splits(blocks, K) if self.force_skinny is None else self.force_skinny[0]
        k_per_split = -(-K // want // 128) * 128 if want > 1 else -(-K // 128) * 128
        n_splits = -(-K // k_per_split)
        nt = -(-M // 8)   # activation tiles of 8 rows
        key = ("gemm_skinny", a.device, nt, n_out, n_splits, gate_up)
        buf = self._scratch.get(key)
        if buf is None:
            floats = blocks * n_splits * (2 if gate_up else 1) * 16 * 8 * nt if n_splits > 1 else 1
            buf = (torch.empty(floats, dtype=torch.float32, device=a.device),
                   torch.zeros(blocks, dtype=torch.int32, device=a.device))
            self._scratch[key] = buf
        stats_out = None
        if add_to is not None:
            out = add_to.x if hasattr(add_to, "stats") else add_to
            if out_float32 or out.dtype != torch.bfloat16 or tuple(out.shape) != (M, n_out) or not out.is_contiguous():
                raise KernelError(f"the product adds to a contiguous bfloat16 [{M}, {n_out}] tensor")
            if out is not add_to:
                stats_out = torch.empty((M, blocks), dtype=torch.float32, device=a.device)
        else:
            out = torch.empty((M, n_out), dtype=torch.float32 if out_float32 else torch.bfloat16, device=a.device)
        warps = self.skinny_warps(blocks * n_splits, -(-M // 8)) if self.force_skinny is None or len(self.force_skinny) < 3 else self.force_skinny[2]
        copy = getattr(w, "_sb_tiled", None)
        if copy is not None and (copy[1] != (2 if gate_up else 1) or (self.force_skinny is not None and not self.force_skinny[1])):
            copy = None   # tiled for the other pairing of rows, or a test asks for the row-major path
        src = copy[0] if copy is not None else w
        tail = (M, n_out, K, n_splits, k_per_split, int(gate_up), int(out_float32), int(copy is not None), warps,
                int(add_to is not None), _ptr(stats_out), _ptr(buf[0]), _ptr(buf[1]), self._stream())
        if act is not None:   # (alpha, limit): the clamped activation in the epilogue of a [gate; up] product
            if not gate_up or norm is not None or add_to is not None or out_float32:
                raise KernelError("the clamped activation sits in the epilogue of a plain [gate; up] product")
            self._check(self.lib.sb_gemm_skinny_gated(_ptr(a), _ptr(src), _ptr(out), M, n_out, K, n_splits, k_per_split,
                                                      int(copy is not None), warps, float(act[0]), float(act[1]), _ptr(buf[0]),
                                                      _ptr(buf[1]), self._stream()), "gemm_skinny_gated")
        elif unary == "relu2":   # the squared relu in the epilogue of a plain product
            if gate_up or norm is not None or add_to is not None or out_float32:
                raise KernelError("an activation sits in the epilogue of a plain product")
            self._check(self.lib.sb_gemm_skinny_relu2(_ptr(a), _ptr(src), _ptr(out), M, n_out, K, n_splits, k_per_split,
                                                      int(copy is not None), warps, _ptr(buf[0]), _ptr(buf[1]), self._stream()),
                        "gemm_skinny_relu2")
        elif unary is not None:   # (a_pos, a_neg): the two-sided activation in the epilogue of a plain product
            if gate_up or norm is not None or add_to is not None or out_float32:
                raise KernelError("the two-sided activation sits in the epilogue of a plain product")
            self._check(self.lib.sb_gemm_skinny_xielu(_ptr(a), _ptr(src), _ptr(out), M, n_out, K, n_splits, k_per_split,
                                                      int(copy is not None), warps, float(unary[0]), float(unary[1]), _ptr(buf[0]),
                                                      _ptr(buf[1]), self._stream()), "gemm_skinny_xielu")
        elif norm is None:
            self._check(self.lib.sb_gemm_skinny(_ptr(a), _ptr(src), _ptr(out), *tail), "gemm_skinny")
        else:
            gamma, eps, stats = norm if len(norm) == 3 else (*norm, None)
            if M > 16 or gamma.dtype != torch.bfloat16 or gamma.numel() != K:
                raise KernelError(f"the norm folded into a product takes up to 16 rows and a bfloat16 weight of {K} values")
            if stats is not None and (stats.dtype != torch.float32 or tuple(stats.shape) != (M, -(-K // 16))):
                raise KernelError(f"the rows' statistics are [{M}, {-(-K // 16)}] floats, not {tuple(stats.shape)} {stats.dtype}")
            self._check(self.lib.sb_gemm_skinny_normed(_ptr(a), _ptr(gamma), float(eps), _ptr(stats), _ptr(src), _ptr(out),
                                                       *tail), "gemm_skinny_normed")
        if stats_out is not None:
            add_to.stats = stats_out
        return out

    def linear_bias(self, a, w, bias):
        """a w^T + bias (32-bit, one per output column); the bias meets the product as it is stored."""
        return self.add_bias(self.linear(a, w), bias)

    def linear(self, a, w, out_float32=False, norm=None, add_to=None):
        """a [M, K] times w [N, K] transposed -> [M, N] in a's dtype, or 32-bit when asked.

        float32: this library's CUDA-core product, always.  bfloat16: the weight-streaming kernels for up
        to 16 rows (and for the output head up to 64), cuBLAS for larger products, the CUDA-core product for what is left.

        norm=(weight, eps[, statistics]): the product of the RMSNorm of a's rows; add_to=x: x += product, in place, x
        returned (see ``_skinny``).  Both for bfloat16 and up to 16 rows: the decode product takes them in its prologue
        and epilogue; ``folds`` says whether that pays."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or a.dtype != w.dtype:
            raise KernelError(f"linear: a is {tuple(a.shape)} {a.dtype}, w is {tuple(w.shape)} {w.dtype}")
        if norm is not None or add_to is not None:
            if not self._can_fold(M, a.dtype, K):
                raise KernelError(f"linear: no folded norm or sum for {M} rows of {K} {a.dtype} values")
            return self._skinny(a, w, N, False, out_float32, norm, add_to)
        if a.dtype == torch.bfloat16 and K % 8 == 0:
            if self._takes_stream(M, N, K, False):
                return self._stream_product(a, w, N, False, out_float32)
            if M <= self.SKINNY_MAX_ROWS:
                return self._skinny(a, w, N, False, out_float32)
            if M * N * K > self.GENERAL_GEMM_MAX_WORK:
                if out_float32:
                    return torch.mm(a, w.t(), out_dtype=torch.float32)
                return torch.mm(a, w.t())
        out = torch.empty((M, N), dtype=torch.float32 if out_float32 else a.dtype, device=a.device)
        self._check(self.lib.sb_gemm_general(_code(a.dtype), int(out_float32 or a.dtype == torch.float32), _ptr(a), _ptr(w),
                                             _ptr(out), M, N, K, self._stream()), "gemm_general")
        return out

    def linear_swiglu(self, h, w_gate_up, norm=None):
        """swiglu(h @ w_gate_up^T) for a fused [gate; up] matrix: [M, K] -> [M, rows / 2].  norm: as in ``linear``."""
        M, K = h.shape
        if norm is not None:
            if not self._can_fold(M, h.dtype, K) or h.dtype != w_gate_up.dtype:
                raise KernelError(f"linear_swiglu: no folded norm for {M} rows of {K} {h.dtype} values")
            return self._skinny(h, w_gate_up, w_gate_up.shape[0] // 2, True, False, norm)
        if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and K % 8 == 0:
            if self._takes_stream(M, w_gate_up.shape[0] // 2, K, True):
                return self._stream_product(h, w_gate_up, w_gate_up.shape[0] // 2, True, False)
            if M <= self.SKINNY_MAX_ROWS:
                return self._skinny(h, w_gate_up, w_gate_up.shape[0] // 2, True, False)
        return self.swiglu(self.linear(h, w_gate_up))

    def linear_gated_clamp(self, h, w_gate_up, alpha, limit):
        """gated_clamp(h @ w_gate_up^T) for a fused [gate; up] matrix: [M, K] -> [M, rows / 2].  For the few rows of a decode
        step the activation sits in the product's epilogue, as SwiGLU does in ``linear_swiglu``."""
        M, K = h.shape
        if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and K % 8 == 0 and M <= self.SKINNY_MAX_ROWS:
            return self._skinny(h, w_gate_up, w_gate_up.shape[0] // 2, True, False, act=(alpha, limit))
        return self.gated_clamp(self.linear(h, w_gate_up), alpha, limit)

    # ---- attention ----------------------------------------------------------------------

    def qk_norm_rope_store(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary):
        dt = _code(qkv.dtype)
        wdt = _code(q_norm.dtype) if q_norm is not None else dt
        if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_store: qkv has the wrong width")
        if head_dim > 512:
            raise KernelError(f"qk_norm_rope_store takes head sizes up to 512, not {head_dim}")
        q = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        cos = sin = None
        rotary_dim = 0
        if rotary is not None:
            cos, sin, rotary_dim = rotary
            if cos.dtype != qkv.dtype or cos.shape[1] * 2 != rotary_dim:
                raise KernelError("qk_norm_rope_store: rotary tables do not fit the run")
            if cos.shape[0] < ctx.kv_bound:
                raise KernelError(f"the rotary table covers {cos.shape[0]} positions, the step reaches {ctx.kv_bound}")
        kv = self._kv(layer_cache)
        if kv.head_dim != head_dim or (n_kv_heads and kv.n_kv_heads != n_kv_heads):
            raise KernelError("qk_norm_rope_store: the layer's cache has other head sizes than the mixer")
        self._check(self.lib.sb_qk_rope_store(dt, wdt, _ptr(qkv), _ptr(q), self._batch(ctx), kv, n_heads, n_kv_heads,
                                              _ptr(q_norm), _ptr(k_norm), eps, _ptr(cos), _ptr(sin), rotary_dim,
                                              _ptr(ctx.status), self._stream()), "qk_rope_store")
        return q

    def sm_count(self) -> int:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    def decode_resident(self, head_dim: int) -> int:
        """Blocks of the split-key decode attention that the GPU holds at once (two per SM at head size 128:
        100 KB of shared memory each)."""
        return (2 if head_dim > 64 else 4) * self.sm_count()

    def decode_splits(self, n_seqs: int, n_kv_heads: int, max_pages: int, head_dim: int = 128) -> int:
        """How many blocks share one (sequence, kv head).  Measured on a B200 at a context of 4,096 with 8 kv heads,
        in the whole decode step (ms a step for splits 2 / 4 / 6 / 8 / 16):
          batch 1 (8 pairs):   - / 2.32 / 2.18 / 2.13 / 2.16        batch 2 (16 pairs): 2.68 / 2.30 / 2.19 / 2.60 / 2.28
          batch 4 (32 pairs): - / 2.38 / 2.41 (5) / 2.79 / 2.71     batch 8 (64 pairs): 2.80 / 2.81 / 3.14 / 3.39 / 3.51
          batch 16 (128 pairs): 2 splits 3.80, 3 splits 4.16        batch 32 (256 pairs): 1 split 5.33, 2 splits 5.50
        About 64 to 128 blocks in all is best while the pairs are few (every block then has an SM and the deeper
        pipeline to itself, and a share pays its fixed costs once: loading the queries, merging the warps, meeting
        the other shares); clusters of 7 or 8 blocks are slow as soon as there are 16 or more of them (7 splits at
        batch 2: 2.65 ms), so beyond 8 pairs a pair has 6 splits at most.  A function of shapes only, so that a
        captured graph stays valid as sequences grow."""
        if os.environ.get("STARTER_B200_ATTN_SPLITS"):   # a tuning override; the kernel refuses what its merge cannot hold
            return max(1, min(int(os.environ["STARTER_B200_ATTN_SPLITS"]), 256))
        pairs = max(n_seqs * n_kv_heads, 1)
        if pairs <= 8:
            want = 8 if max_pages <= 96 else 16     # a cache of 16,384 tokens a sequence: 2.44 ms with 16, 2.65 with 8
        elif pairs <= 16:
            want = 6
        elif pairs <= 32:
            want = 4
        elif pairs <= 64:
            want = 4 if max_pages <= 96 else 2      # batch 8 at 16,384 tokens: 4.83 ms with 2, 4.99 with 4, 5.78 with 8
        else:
            want = 256 // pairs
        return max(1, min(want, max_pages, self.decode_resident(head_dim) // pairs))

    def _decode_scratch(self, device, n_seqs, n_heads, n_kv_heads, head_dim, n_splits):
        key = ("attn_decode", device, n_seqs, n_heads, n_kv_heads, head_dim, n_splits)
        buf = self._scratch.get(key)
        if buf is None:
            floats = max(n_seqs * n_heads * n_splits * (head_dim + 2), 1)
            buf = (torch.empty(floats, dtype=torch.float32, device=device),
                   torch.zeros(n_seqs * n_kv_heads, dtype=torch.int32, device=device))
            self._scratch[key] = buf
        return buf

    def _decode_route(self, ctx, kv, n_heads):
        """Which decode kernel serves a step of one token per sequence (bfloat16 cache with head size 64 or 128, at most
        16 query heads per kv head): "split" (a grid of (sequence, kv head, split), the blocks handed out by the
        hardware as others end) or "balanced" (one block per SM, equal shares of all pages, worked out on the device
        from the lengths); None when the step is of another kind.

        Measured alone at 4B sizes with sequences of equal length (us, balanced / split with one block per pair):
        batch 64 at context 2,048: 95.8 / 87.9, at 4,096: 168.3 / 163.8; batch 128 at 2,048: 175 / 169; batch 256 at 1,024:
        191 / 173; in the step at batch 64: 8.50 / 8.36 ms.  The balanced kernel pays ~6 us before its first page and its
        blocks end up to 10 us apart; blocks handed out one by one even that out by themselves.  With very unequal
        lengths (``ctx.uneven``: the longest sequence more than three times the mean) the split kernel, whose blocks per
        pair are a matter of shapes, leaves the longest sequence to a few blocks, and the balanced kernel takes over at
        every batch size.  One sequence of 16,384 tokens among others of 256 (us, split / balanced): batch 8: 81 / 27,
        batch 16: 83 / 34, batch 32: 153 / 41, batch 64: 162 / 43; one of 4,096: 18 / 20, 27 / 21, 45 / 28, 53 / 34."""
        if kv.head_dim not in (64, 128) or n_heads % kv.n_kv_heads or n_heads // kv.n_kv_heads > 16:
            return None
        if not (ctx.max_q_len == 1 and ctx.n_rows == ctx.n_seqs):
            return None
        if self.force_decode_route is not None:
            return self.force_decode_route
        if self.decode_balanced and getattr(ctx, "uneven", False) and ctx.n_seqs <= 1024:
            return "balanced"
        return "split"

    def uneven_matters(self, n_seqs: int) -> bool:
        """Whether a decode step of this many sequences would run other kernels when its context says ``uneven``
        (so that a caller who keeps captured graphs need not keep two alike)."""
        return self.force_decode_route is None and self.decode_balanced and 2 <= n_seqs <= 1024

    def _split_decode(self, ctx, kv, n_heads) -> bool:
        return self._decode_route(ctx, kv, n_heads) == "split"

    def _balanced_scratch(self, device, ctx, kv, n_heads):
        grid = min(self.sm_count(), 512)
        key = ("attn_decode_balanced", device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, grid)
        buf = self._scratch.get(key)
        if buf is None:
            pairs = ctx.n_seqs * kv.n_kv_heads
            floats = (pairs + grid) * (n_heads // kv.n_kv_heads) * (kv.head_dim + 2)
            buf = self._scratch[key] = (torch.empty(floats, dtype=torch.float32, device=device),
                                        torch.zeros(pairs, dtype=torch.int32, device=device))
        return grid, buf

    def qk_attention(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary, scale, window,
                     then=None):
        """qk_norm_rope_store and attention in one kernel, for the steps that the split-key decode kernel serves and a
        rotary encoding over the whole head (or none).  Returns None when the step is not of that kind: the caller then
        makes the two calls."""
        if not self.fuse_qk or qkv.dtype != torch.bfloat16 or layer_cache.group.k.dtype != torch.bfloat16:
            return None
        kv = self._kv(layer_cache)
        route = self._decode_route(ctx, kv, n_heads)
        if kv.head_dim != head_dim or (n_kv_heads and kv.n_kv_heads != n_kv_heads) or route is None:
            return None
        if route == "balanced" and not self.fuse_qk_balanced:
            return None
        if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("qk_attention: qkv has the wrong width")
        cos = sin = None
        if rotary is not None:
            cos, sin, rotary_dim = rotary
            if rotary_dim != head_dim or cos.dtype != torch.bfloat16:
                return None
            if cos.shape[1] * 2 != rotary_dim:
                raise KernelError("qk_attention: rotary tables do not fit the run")
            if cos.shape[0] < ctx.kv_bound:
                raise KernelError(f"the rotary table covers {cos.shape[0]} positions, the step reaches {ctx.kv_bound}")
        norm_f32 = 0
        for w in (q_norm, k_norm):
            if w is not None:
                if w.dtype not in (torch.float32, torch.bfloat16):
                    return None
                norm_f32 = int(w.dtype == torch.float32)
        if q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype:
            return None
        # `then`: the matrix that the next product streams; the kernel asks for it into L2 as it finishes its keys
        next_w, next_bytes = None, 0
        if then is not None and self.prefetch_next_bytes > 0 and then.dtype == torch.bfloat16:
            copy = getattr(then, "_sb_tiled", None)
            src = copy[0] if copy is not None and ctx.n_rows <= self.SKINNY_MAX_ROWS else then
            next_w, next_bytes = c_void_p(src.data_ptr()), min(src.numel() * 2, self.prefetch_next_bytes) & ~15
        fused = SbFusedQK(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin), _ptr(ctx.status), float(eps), norm_f32,
                          int(n_kv_heads > 0), 0, next_w, next_bytes)
        out = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        if route == "balanced":
            grid, buf = self._balanced_scratch(qkv.device, ctx, kv, n_heads)
            self._check(self.lib.sb_attn_decode_balanced_fused(fused, _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                               int(window or 0), grid, _ptr(buf[0]), _ptr(buf[1]),
                                                               self._stream()), "attn_decode_balanced_fused")
            return out
        n_splits = self.decode_splits(ctx.n_seqs, kv.n_kv_heads, layer_cache.group.table_width, kv.head_dim)
        partial, counters = self._decode_scratch(qkv.device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, n_splits)
        self._check(self.lib.sb_attn_decode_fused(fused, _ptr(out), self._batch(ctx), kv, n_heads, scale, int(window or 0),
                                                  n_splits, _ptr(partial), _ptr(counters), self._stream()), "attn_decode_fused")
        return out

    def attention(self, ctx, q, layer_cache, n_heads, scale, window):
        """Causal attention of the step's rows over the layer's cache.  bfloat16 with head size 64 or
        128: the split-key decode kernel for steps of one token per sequence, the flash kernel for
        everything else.  Other head sizes and float32 take the general kernel."""
        out = torch.empty_like(q)
        kv = self._kv(layer_cache)
        if kv.head_dim > 256:
            raise KernelError(f"attention takes head sizes up to 256, not {kv.head_dim}")
        if n_heads % kv.n_kv_heads:
            raise KernelError(f"{n_heads} query heads cannot share {kv.n_kv_heads} key/value heads evenly")
        if q.dtype == torch.bfloat16 and kv.head_dim in (64, 128):
            decode = ctx.max_q_len == 1 and ctx.n_rows == ctx.n_seqs and n_heads // kv.n_kv_heads <= 16
            split = decode and self._split_decode(ctx, kv, n_heads)
            if decode and not split:
                # More pairs than blocks fit at once: one block per SM, each with an equal share of all pages.
                grid, buf = self._balanced_scratch(q.device, ctx, kv, n_heads)
                self._check(self.lib.sb_attn_decode_balanced(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                             int(window or 0), grid, _ptr(buf[0]), _ptr(buf[1]),
                                                             self._stream()), "attn_decode_balanced")
            elif split:
                g = layer_cache.group
                n_splits = self.decode_splits(ctx.n_seqs, kv.n_kv_heads, g.table_width, kv.head_dim)
                partial, counters = self._decode_scratch(q.device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, n_splits)
                self._check(self.lib.sb_attn_decode(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                    int(window or 0), n_splits, _ptr(partial), _ptr(counters),
                                                    self._stream()), "attn_decode")
            elif (self.prefill_tensor_memory and kv.head_dim == 128
                  and ctx.max_q_len * (n_heads // kv.n_kv_heads) >= 128):
                # long pieces at head size 128: the tcgen05 kernel (S and O in tensor memory, TMA for keys and values)
                self._check(self.lib.sb_attn_prefill_tc(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                        int(window or 0), ctx.max_q_len, layer_cache.group.pool_pages + 1,
                                                        _ptr(self.kernel_status(q.device)), self._stream()), "attn_prefill_tc")
            else:
                self._check(self.lib.sb_attn_prefill(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                     int(window or 0), ctx.max_q_len, self._stream()), "attn_prefill")
            return out
        self._check(self.lib.sb_attention_general(_code(q.dtype), _ptr(q), _ptr(out), self._batch(ctx), kv,
                                                  n_heads, scale, int(window or 0), self._stream()), "attention_general")
        return out

    # ---- attention with options, latents, the linear recurrence --------------------------

    HEADS_LIBRARY_MIN_ROWS = 64

    def linear_heads(self, a, w, out):
        """out[m, h, :] = a[m, h, :] times w[h] transposed, for views a [rows, heads, K] and out [rows, heads, N] whose
        last axis is contiguous (a head's columns inside wider rows) and w [heads, N, K]."""
        rows, H, K = a.shape
        N = w.shape[1]
        if (tuple(w.shape) != (H, N, K) or tuple(out.shape) != (rows, H, N) or a.stride(2) != 1 or out.stride(2) != 1
                or not w.is_contiguous() or not (a.dtype == w.dtype == out.dtype)):
            raise KernelError(f"linear_heads: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if a.dtype == torch.bfloat16 and rows > self.HEADS_LIBRARY_MIN_ROWS and K % 8 == 0 and N % 8 == 0:
            # many rows: the library's batched product on the tensor cores, as the plain products of a prompt
            out.copy_(torch.bmm(a.transpose(0, 1), w.transpose(1, 2)).transpose(0, 1))
            return out
        self._check(self.lib.sb_gemm_heads(_code(a.dtype), _ptr(a), a.stride(0), a.stride(1), _ptr(w), _ptr(out), out.stride(0),
                                           out.stride(1), rows, N, K, H, self._stream()), "gemm_heads")
        return out

    def _flex(self, layer_cache, q=None, n_heads=0, scale=1.0, v_dim=None, values_in_keys=False, sink=None, head_scale=None,
              slopes=None, chunk=None, window=None, keep_first=0, softcap=None, talk=None) -> SbFlex:
        g = layer_cache.group
        k = layer_cache.k
        if values_in_keys:
            v, v_row = k, g.request.head_dim
            v_dim = g.request.head_dim if v_dim is None else v_dim
        else:
            v, v_row = layer_cache.v, g.v_dim
            v_dim = g.v_dim if v_dim is None else v_dim
            if v is None or v_dim != g.v_dim:
                raise KernelError("the layer's cache keeps no values of this width")
        if v_dim > v_row:
            raise KernelError("values wider than the rows they are read from")
        for t in (sink, head_scale, slopes):
            if t is not None and (t.dtype != torch.float32 or t.numel() != n_heads or not t.is_contiguous()):
                raise KernelError("per-head numbers of the attention are 32-bit, one per query head")
        return SbFlex(_ptr(q), q.stride(0) if q is not None else 0, q.stride(1) if q is not None else 0, _ptr(k), _ptr(v),
                      g.table.data_ptr(), _ptr(head_scale), _ptr(slopes), _ptr(sink), g.table_width, g.ring_pages, n_heads,
                      g.request.num_kv_heads, g.request.head_dim, v_dim, v_row, int(window or 0), int(chunk or 0), float(scale),
                      0 if values_in_keys else g.v_heads, g.pinned_pages, int(keep_first or 0), float(softcap or 0.0), _ptr(talk))

    def flex_attention(self, ctx, q, layer_cache, scale, v_dim, values_in_keys=False, sink=None, head_scale=None, slopes=None,
                       chunk=None, window=None):
        """Causal attention of the step's rows, q a view [rows, heads, key width] (last axis contiguous), over the
        layer's cache -> [rows, heads * v_dim].  score = q.k * scale * head_scale[h] - slopes[h] * distance; ``chunk``
        and ``window`` narrow what a row sees; ``sink`` [heads] adds exp(sink_h) to the softmax's denominator;
        ``values_in_keys``: the values are the first v_dim columns of the key rows."""
        rows, H, kd = q.shape
        if q.stride(2) != 1 or kd != layer_cache.group.request.head_dim or q.dtype != layer_cache.k.dtype:
            raise KernelError(f"flex_attention: q {tuple(q.shape)} {q.dtype} does not fit the layer's cache")
        if H % layer_cache.group.request.num_kv_heads:
            raise KernelError(f"{H} query heads cannot share {layer_cache.group.request.num_kv_heads} key/value heads evenly")
        if layer_cache.group.pinned_pages:
            raise KernelError("flex_attention: a cache that pins a sequence's first pages is read by talking_attention")
        p = self._flex(layer_cache, q, H, scale, v_dim, values_in_keys, sink, head_scale, slopes, chunk, window)
        out = torch.empty((rows, H * v_dim), dtype=q.dtype, device=q.device)
        if v_dim > 1024:
            raise KernelError(f"attention takes values of up to 1024 columns, not {v_dim}")
        if self._flex_takes_rows64(ctx, q, p, values_in_keys):
            self._check(self.lib.sb_flex_attention_rows64(p, self._batch(ctx), _ptr(out), ctx.max_q_len, int(values_in_keys),
                                                          self._stream()), "flex_attention_rows64")
            return out
        if self._flex_takes_mma(q, p, values_in_keys):
            n_splits = self.flex_splits(ctx, p, layer_cache.group.table_width)
            partial = None
            if n_splits > 1:
                key = ("flex_partial", q.device, rows, H, n_splits, v_dim)
                partial = self._scratch.get(key)
                if partial is None:
                    partial = self._scratch[key] = torch.empty(rows * H * n_splits * (v_dim + 2), dtype=torch.float32, device=q.device)
            self._check(self.lib.sb_flex_attention_mma(p, self._batch(ctx), _ptr(out), ctx.max_q_len, n_splits, _ptr(partial),
                                                       int(values_in_keys), self._stream()), "flex_attention_mma")
            if n_splits > 1:
                self.launches += 1   # the merge of the splits
            return out
        self._check(self.lib.sb_flex_attention_general(_code(q.dtype), p, self._batch(ctx), _ptr(out), self._stream()),
                    "flex_attention_general")
        return out

    MAX_BLOCK_SHARED = 227 * 1024

    def _flex_takes_mma(self, q, p: SbFlex, values_in_keys: bool) -> bool:
        """The tensor-core kernel takes bfloat16, key widths that are multiples of 16, values of 64, 128, 256 or 512
        columns, 1, 2, 4, 8 or a multiple of 16 query heads per key/value head, and rows it can fetch 16 bytes at a
        time; the warp-per-row kernel serves everything else (and every 32-bit run)."""
        if not self.flex_tensor_cores or q.dtype != torch.bfloat16:
            return False
        smem = self.lib.sb_flex_attention_mma_smem(p.k_dim, p.v_dim, p.n_heads // p.n_kv_heads, int(values_in_keys))
        if smem < 0 or smem > self.MAX_BLOCK_SHARED:
            return False
        return q.stride(0) % 8 == 0 and q.stride(1) % 8 == 0 and q.data_ptr() % 16 == 0 and p.v_row % 8 == 0

    FLEX_PROMPT_MIN_ROWS = 32

    def _flex_takes_rows64(self, ctx, q, p: SbFlex, values_in_keys: bool) -> bool:
        """The kernel for prompts (64 rows per block, a warp per 16 rows, no meeting of warps inside a page) takes steps
        whose sequences bring at least 32 rows of scores per key/value head, values of 64 or 128 columns and a number of
        heads per key/value head that divides 64; the rest of what the tensor-core path takes goes to the 16-row kernel."""
        if not self.flex_tensor_cores or q.dtype != torch.bfloat16:
            return False
        per_kv = p.n_heads // p.n_kv_heads
        if ctx.max_q_len * per_kv < self.FLEX_PROMPT_MIN_ROWS:
            return False
        smem = self.lib.sb_flex_attention_rows64_smem(p.k_dim, p.v_dim, per_kv, int(values_in_keys))
        if smem < 0 or smem > self.MAX_BLOCK_SHARED:
            return False
        return q.stride(0) % 8 == 0 and q.stride(1) % 8 == 0 and q.data_ptr() % 16 == 0 and p.v_row % 8 == 0

    def flex_splits(self, ctx, p: SbFlex, max_pages: int) -> int:
        """Blocks along the keys per (sequence, key/value head) in a step of one token per sequence: enough for two
        blocks per SM, none with less than two pages.  A function of shapes only, so that a captured graph stays valid."""
        if ctx.max_q_len != 1:
            return 1
        per_kv = p.n_heads // p.n_kv_heads
        blocks = ctx.n_seqs * p.n_kv_heads * max(1, per_kv // 16)
        reach = max_pages
        for r in (p.window, p.chunk):
            if r:
                reach = min(reach, r // 64 + 2)
        return max(1, min(-(-2 * self.sm_count() // blocks), reach // 2, 64))

    def kv_store(self, ctx, k, v, layer_cache, value_norm_eps=None):
        """The step's keys [rows, kv_heads * key width] and values [rows, kv_heads * value width] (views of wider rows
        will do) into the layer's cache; with ``value_norm_eps`` every head's value is divided by its root mean square."""
        g = layer_cache.group
        G = g.request.num_kv_heads
        if (k.shape[1] != G * g.request.head_dim or v.shape[1] != G * g.v_dim or k.stride(1) != 1 or v.stride(1) != 1
                or k.dtype != layer_cache.k.dtype or v.dtype != k.dtype or g.v_heads != G):
            raise KernelError("kv_store: keys or values do not fit the layer's cache")
        p = self._flex(layer_cache)
        self._check(self.lib.sb_kv_store(_code(k.dtype), _ptr(k), k.stride(0), _ptr(v), v.stride(0), self._batch(ctx), p,
                                         int(value_norm_eps is not None), float(value_norm_eps or 0.0), _ptr(ctx.status),
                                         self._stream()), "kv_store")

    def rotate_pairs(self, ctx, src, dst, freqs, rot):
        """dst = src [rows, heads, cols] (views, last axis contiguous) with the first ``rot`` columns of every head
        turned in neighbouring pairs by the row's position times ``freqs`` (32-bit, [rot / 2])."""
        rows, H, cols = src.shape
        if tuple(dst.shape) != (rows, H, cols) or src.stride(2) != 1 or dst.stride(2) != 1 or src.dtype != dst.dtype:
            raise KernelError("rotate_pairs: source and destination differ")
        if freqs is None:
            rot = 0
        elif freqs.dtype != torch.float32 or freqs.numel() * 2 != rot:
            raise KernelError("rotate_pairs: one 32-bit frequency per pair")
        self._check(self.lib.sb_rotate_pairs(_code(src.dtype), _ptr(src), src.stride(0), src.stride(1), _ptr(dst), dst.stride(0),
                                             dst.stride(1), self._batch(ctx), _ptr(freqs), H, cols, int(rot), self._stream()),
                    "rotate_pairs")

    def latent_prepare(self, ctx, down, layer_cache, q_rank, kv_rank, rot_dim, q_norm, kv_norm, eps, freqs, rot, rows_too=False):
        """down [rows, q_rank + kv_rank + rot_dim] -> the normed query latent [rows, q_rank]; the normed key/value
        latent and the rotated shared part go to the row's place in the layer's cache.  ``rows_too``: what went to the
        cache is returned as well, (cq, [rows, kv_rank + rot_dim])."""
        if down.shape[1] != q_rank + kv_rank + rot_dim or not down.is_contiguous() or q_norm.dtype != kv_norm.dtype:
            raise KernelError("latent_prepare: the down-projection has the wrong width")
        if down.dtype == torch.float32 and q_norm.dtype != torch.float32:
            raise KernelError("a float32 run needs float32 norm weights")
        if freqs is None:
            rot = 0
        p = self._flex(layer_cache, values_in_keys=True)
        cq = torch.empty((down.shape[0], q_rank), dtype=down.dtype, device=down.device)
        kept = torch.empty((down.shape[0], kv_rank + rot_dim), dtype=down.dtype, device=down.device) if rows_too else None
        self._check(self.lib.sb_latent_prepare(_code(down.dtype), _code(q_norm.dtype), _ptr(down), _ptr(cq), self._batch(ctx), p,
                                               q_rank, kv_rank, rot_dim, _ptr(q_norm), _ptr(kv_norm), float(eps), _ptr(freqs),
                                               int(rot), _ptr(ctx.status), _ptr(kept), self._stream()), "latent_prepare")
        return (cq, kept) if rows_too else cq

    def token_shift(self, ctx, h, state, prev_offset, mu):
        """[n, rows, width]: h + (h' - h) * mu[m] for every row of mu, h' the row before (for a sequence's first row of
        the step: what its record in ``state`` [slots, floats] holds from ``prev_offset`` on)."""
        rows, width = h.shape
        if state.dtype != torch.float32 or mu.shape[1] != width or not h.is_contiguous() or not mu.is_contiguous():
            raise KernelError("token_shift: a 32-bit state record and one blend vector per output")
        out = torch.empty((mu.shape[0], rows, width), dtype=h.dtype, device=h.device)
        self._check(self.lib.sb_token_shift(_code(h.dtype), _code(mu.dtype), _ptr(h), _ptr(state), state.stride(0), int(prev_offset),
                                            _ptr(mu), mu.shape[0], self._batch(ctx), width, _ptr(out), self._stream()),
                    "token_shift")
        return out

    def wkv_scan(self, ctx, r, k, v, g, decay_pre, w0, u, norm, eps, h, state, heads, dim, prev_offset):
        """The recurrence over every sequence's rows, from and back into ``state``; returns the heads' outputs after the
        unit norm, the scale and the gate [rows, heads * dim].  Also leaves each sequence's last row of h in its record."""
        inner = heads * dim
        if dim > 4096:
            raise KernelError(f"the recurrence takes heads of up to 4096 channels, not {dim}")
        for t in (r, k, v, g):
            if tuple(t.shape) != (h.shape[0], inner) or not t.is_contiguous() or t.dtype != h.dtype:
                raise KernelError("wkv_scan: r, k, v, g are contiguous [rows, heads * dim] in the run's dtype")
        for t in (decay_pre, w0, u, norm):
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise KernelError("wkv_scan: decay, bonus and norm weights are 32-bit")
        y = torch.empty((h.shape[0], inner), dtype=h.dtype, device=h.device)
        self._check(self.lib.sb_wkv_scan(_code(h.dtype), _ptr(r), _ptr(k), _ptr(v), _ptr(g), _ptr(decay_pre), _ptr(w0), _ptr(u),
                                         _ptr(norm), float(eps), _ptr(h), h.shape[1], _ptr(state), state.stride(0),
                                         int(prev_offset), self._batch(ctx), heads, dim, _ptr(y), self._stream()), "wkv_scan")
        return y

    # ---- a residual in streams, two-map attention, gated linear attention, experts -------

    def embed_streams(self, tokens, table, status, scale, copies):
        """[rows, copies * width] 32-bit: the table's rows by token id, times ``scale``, ``copies`` times side by side."""
        out = torch.empty((tokens.shape[0], copies * table.shape[1]), dtype=torch.float32, device=table.device)
        self._check(self.lib.sb_embed_streams(_code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0],
                                              table.shape[1], table.shape[0], 1.0 if scale is None else float(scale), int(copies),
                                              _ptr(status), self._stream()), "embed_streams")
        return out

    def stream_norm(self, x, streams, pending, read_w, weight, eps, out_dtype):
        """x [rows, streams * width] 32-bit, in place: with ``pending`` = (y, mix [S, S], out [S]) every stream first becomes
        X'_t = sum_s mix[s, t] X_s + out[t] y; then, with ``read_w`` [S], RMSNorm(sum_s read_w[s] X'_s) * weight is returned
        in ``out_dtype`` (None without ``read_w``)."""
        rows, S = x.shape[0], int(streams)
        width = x.shape[1] // S
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != S * width or not 1 <= S <= 8:
            raise KernelError("the streams are 32-bit, contiguous, one to eight copies side by side")
        y = mix = out_w = None
        if pending is not None:
            y, mix, out_w = pending
            if (y.dtype != out_dtype or tuple(y.shape) != (rows, width) or not y.is_contiguous() or mix.dtype != torch.float32
                    or out_w.dtype != torch.float32 or mix.numel() != S * S or out_w.numel() != S or not mix.is_contiguous()):
                raise KernelError("a branch output has the run's dtype and one stream's shape; its return weights are 32-bit")
        n = None
        if read_w is not None:
            if read_w.dtype != torch.float32 or read_w.numel() != S or weight.numel() != width:
                raise KernelError("a stream read takes one 32-bit weight per stream and a norm weight per column")
            if out_dtype == torch.float32 and weight.dtype != torch.float32:
                raise KernelError("a float32 run needs float32 norm weights")
            n = torch.empty((rows, width), dtype=out_dtype, device=x.device)
        self._check(self.lib.sb_stream_norm(_code(out_dtype), _code(weight.dtype) if weight is not None else _code(out_dtype), _ptr(x),
                                            _ptr(y), _ptr(mix), _ptr(out_w), _ptr(read_w), _ptr(weight), _ptr(n), rows, width, S,
                                            float(eps), self._stream()), "stream_norm")
        return n

    def rotate_half_store(self, ctx, q, k, v, layer_cache, freqs, rot, magnitude):
        """q [rows, nq, D], k [rows, key heads, D] (views of wider rows, heads side by side) with the first ``rot`` columns
        of every head turned (column i with column i + rot / 2) by position * ``freqs`` (32-bit, [rot / 2]), cosines and
        sines times ``magnitude``; the turned keys and v [rows, value heads * value width] go to the layer's cache, the
        turned queries are returned [rows, nq, D]."""
        g = layer_cache.group
        rows, nq, D = q.shape
        if (D != g.request.head_dim or tuple(k.shape) != (rows, g.request.num_kv_heads, D) or v.shape[1] != g.v_heads * g.v_dim
                or q.stride(2) != 1 or k.stride(2) != 1 or v.stride(1) != 1 or q.stride(1) != D or k.stride(1) != D
                or not (q.dtype == k.dtype == v.dtype == layer_cache.k.dtype)):
            raise KernelError("rotate_half_store: queries, keys or values do not fit the layer's cache")
        if freqs is None:
            rot = 0
        elif freqs.dtype != torch.float32 or freqs.numel() * 2 != rot or rot > D:
            raise KernelError("rotate_half_store: one 32-bit frequency per pair of turned columns")
        p = self._flex(layer_cache)
        out = torch.empty((rows, nq, D), dtype=q.dtype, device=q.device)
        self._check(self.lib.sb_rotate_half_store(_code(q.dtype), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0),
                                                  _ptr(out), self._batch(ctx), p, _ptr(freqs), int(rot), float(magnitude), nq,
                                                  _ptr(ctx.status), self._stream()), "rotate_half_store")
        return out

    def diff_combine(self, a, heads, kv_heads, v_dim, lam, eps, post, gate=None):
        """a [rows, 2 * heads * v_dim], the two maps of every head in the order (key/value head, map, head of the group) ->
        [rows, heads * v_dim]: (a1 - lam * a2) / sqrt(mean(.^2) + eps) * post, head by head.  ``gate`` [rows, heads * v_dim]
        (a view of wider rows will do): the result times sigmoid(gate), element by element."""
        rows = a.shape[0]
        if a.shape[1] != 2 * heads * v_dim or not a.is_contiguous() or heads % kv_heads:
            raise KernelError("diff_combine: two maps of v_dim columns per head")
        if gate is not None and (tuple(gate.shape) != (rows, heads * v_dim) or gate.stride(1) != 1 or gate.dtype != a.dtype):
            raise KernelError("diff_combine: the gate has one column per output column, in the run's dtype")
        out = torch.empty((rows, heads * v_dim), dtype=a.dtype, device=a.device)
        self._check(self.lib.sb_diff_combine(_code(a.dtype), _ptr(a), _ptr(out), rows, heads, kv_heads, v_dim, float(lam), float(eps),
                                             float(post), _ptr(gate), gate.stride(0) if gate is not None else 0, self._stream()),
                    "diff_combine")
        return out

    # ---- layers in passes, mixers side by side, keys as values, the matrix memory ----------

    def add_rows(self, x, rows_too=None, vector=None, out=None):
        """x + rows_too + vector over 32-bit rows [rows, width] (either addend may be None); into ``out`` (x itself will
        do), else into a new tensor."""
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("add_rows: contiguous 32-bit rows")
        if rows_too is not None and (rows_too.dtype != torch.float32 or rows_too.shape != x.shape or not rows_too.is_contiguous()):
            raise KernelError("add_rows: the rows that are added have the shape and type of the others")
        if vector is not None and (vector.dtype != torch.float32 or vector.numel() != x.shape[1] or not vector.is_contiguous()):
            raise KernelError("add_rows: one 32-bit number per column")
        if out is None:
            out = torch.empty_like(x)
        self._check(self.lib.sb_add_rows(_ptr(x), _ptr(rows_too), _ptr(vector), _ptr(out), x.shape[0], x.shape[1], self._stream()),
                    "add_rows")
        return out

    def add_bias(self, y, bias):
        """y += bias (32-bit, one per column), in place; the sum is 32-bit and rounded once."""
        if not y.is_contiguous() or bias.dtype != torch.float32 or bias.numel() != y.shape[1]:
            raise KernelError("add_bias: contiguous rows and one 32-bit number per column")
        self._check(self.lib.sb_add_bias(_code(y.dtype), _ptr(y), _ptr(bias), y.shape[0], y.shape[1], self._stream()), "add_bias")
        return y

    def scaled_sum(self, a, sa, b, sb):
        """sa * a + sb * b, element by element, 32-bit and rounded once."""
        if a.shape != b.shape or a.dtype != b.dtype or not a.is_contiguous() or not b.is_contiguous():
            raise KernelError("scaled_sum: two contiguous tensors of one shape and type")
        out = torch.empty_like(a)
        self._check(self.lib.sb_scaled_sum(_code(a.dtype), _ptr(a), float(sa), _ptr(b), float(sb), _ptr(out), a.numel(), self._stream()),
                    "scaled_sum")
        return out

    def relu2(self, z):
        if not z.is_contiguous():
            raise KernelError("relu2: a contiguous tensor")
        out = torch.empty_like(z)
        self._check(self.lib.sb_relu2(_code(z.dtype), _ptr(z), _ptr(out), z.numel(), self._stream()), "relu2")
        return out

    def linear_relu2(self, h, w_up):
        """max(h @ w_up^T, 0)^2.  For the few rows of a decode step the activation sits in the product's epilogue."""
        M, K = h.shape
        if h.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and K % 8 == 0 and M <= self.SKINNY_MAX_ROWS:
            return self._skinny(h, w_up, w_up.shape[0], False, False, unary="relu2")
        return self.relu2(self.linear(h, w_up))

    def conv_qk_store(self, ctx, q, k, layer_cache, state, n_heads, q_bias, k_bias, q_conv, k_conv, q_norm, k_norm, eps,
                      temp_coef, temp_every):
        """q [rows, heads * D], k [rows, kv heads * D] (views of wider rows): plus their biases, through a short causal
        convolution per channel (``q_conv`` [heads * D, taps]; ``state`` [slots, taps - 1, (heads + kv heads) * D] holds each
        sequence's last biased projections and is brought up to date), normed per head with the weights of D values, the
        queries times 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1).  The normed keys go to the cache's key rows,
        the keys before the norm to its value rows; the queries come back as [rows, heads, D].  Biases, convolutions and the
        norm weights may be None; ``temp_every`` 0 leaves the queries as they are."""
        g = layer_cache.group
        G, D = g.request.num_kv_heads, g.request.head_dim
        rows = q.shape[0]
        if (tuple(q.shape) != (rows, n_heads * D) or tuple(k.shape) != (rows, G * D) or q.stride(1) != 1 or k.stride(1) != 1
                or q.dtype != layer_cache.k.dtype or k.dtype != q.dtype or g.v_dim != D or g.v_heads != G):
            raise KernelError("conv_qk_store: queries or keys do not fit the layer's cache (its values are as wide as its keys)")
        taps = 0
        if q_conv is not None:
            taps = q_conv.shape[1]
            if (tuple(q_conv.shape) != (n_heads * D, taps) or tuple(k_conv.shape) != (G * D, taps) or q_conv.dtype != torch.float32
                    or k_conv.dtype != torch.float32 or not q_conv.is_contiguous() or not k_conv.is_contiguous()):
                raise KernelError("conv_qk_store: 32-bit convolution weights [channels, taps]")
            if taps > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, (n_heads + G) * D)
                             or not state.is_contiguous()):
                raise KernelError(f"conv_qk_store: the state is [slots, {taps - 1}, {(n_heads + G) * D}] 32-bit numbers")
        for t, n in ((q_bias, n_heads * D), (k_bias, G * D), (q_norm, D), (k_norm, D)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
                raise KernelError("conv_qk_store: biases and norm weights are 32-bit")
        if (q_norm is None) != (k_norm is None):
            raise KernelError("conv_qk_store: queries and keys are normed together or not at all")
        out = torch.empty((rows, n_heads, D), dtype=q.dtype, device=q.device)
        p = self._flex(layer_cache)
        self._check(self.lib.sb_conv_qk_store(_code(q.dtype), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(q_bias), _ptr(k_bias),
                                              _ptr(q_conv), _ptr(k_conv), int(taps), _ptr(state) if taps > 1 else None,
                                              state.stride(0) if taps > 1 else 0, _ptr(q_norm), _ptr(k_norm), float(eps),
                                              float(temp_coef), int(temp_every), _ptr(out), self._batch(ctx), p, n_heads,
                                              _ptr(ctx.status), self._stream()), "conv_qk_store")
        if taps > 1:
            self.launches += 1   # the state's kernel
        return out

    def head_gate(self, a, z, z_col, heads, scale=1.0, out=None):
        """a [rows, heads * V] times sigmoid(z[:, z_col + head]) (z 32-bit, [rows, any]) times ``scale``; into ``out`` (a
        view [rows, heads * V] of wider rows will do) or a new tensor."""
        rows, width = a.shape
        if width % heads or not a.is_contiguous() or z.dtype != torch.float32 or z.stride(1) != 1 or z_col + heads > z.shape[1]:
            raise KernelError("head_gate: contiguous rows of whole heads and 32-bit gates")
        if out is None:
            out = torch.empty_like(a)
        elif tuple(out.shape) != (rows, width) or out.stride(1) != 1 or out.dtype != a.dtype:
            raise KernelError("head_gate: the output has the input's shape and type")
        self._check(self.lib.sb_head_gate(_code(a.dtype), _ptr(a), _ptr(z), z.stride(0), int(z_col), _ptr(out), out.stride(0), rows,
                                          heads, width // heads, float(scale), self._stream()), "head_gate")
        return out

    def mlstm_scan(self, ctx, q, k, v, g, z, i_col, f_col, i_bias, f_bias, cap, norm, eps, q_scale, state, heads, dim, vdim,
                   out_scale=1.0, out=None):
        """The matrix memory's recurrence over every sequence's rows, from and back into ``state`` [slots, heads * dim * vdim
        + heads * dim + heads] (S, the normaliser n, the running maximum m); q, k [rows, heads * dim] and v, g [rows, heads *
        vdim] are views of the same wider rows; z [rows, any] 32-bit holds head h's input gate at column i_col + h and its
        forget gate at f_col + h, before bias, cap and logsigmoid.  Returns the heads' outputs divided by their
        normaliser, unit-normed per head, times ``norm`` [heads * vdim], sigmoid(g) and ``out_scale``; into ``out`` when given
        (a view [rows, heads * vdim] of wider rows)."""
        rows = q.shape[0]
        ld = q.stride(0)
        for t, w in ((q, heads * dim), (k, heads * dim), (v, heads * vdim), (g, heads * vdim)):
            if tuple(t.shape) != (rows, w) or t.stride(1) != 1 or t.stride(0) != ld or t.dtype != q.dtype:
                raise KernelError("mlstm_scan: q, k, v, g are views of rows with one stride, in the run's dtype")
        for t in (i_bias, f_bias, norm, state):
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise KernelError("mlstm_scan: gate biases, norm weight and state are 32-bit and contiguous")
        if (z.dtype != torch.float32 or z.stride(1) != 1 or max(i_col, f_col) + heads > z.shape[1] or z.shape[0] != rows
                or state.shape[1] != heads * dim * vdim + heads * dim + heads or norm.numel() != heads * vdim
                or i_bias.numel() != heads or f_bias.numel() != heads):
            raise KernelError("mlstm_scan: sizes do not fit")
        if out is None:
            y = torch.empty((rows, heads * vdim), dtype=q.dtype, device=q.device)
        elif tuple(out.shape) != (rows, heads * vdim) or out.stride(1) != 1 or out.dtype != q.dtype:
            raise KernelError("mlstm_scan: the output has one column per head and value channel, in the run's dtype")
        else:
            y = out
        raw = torch.empty((rows, heads * vdim), dtype=torch.float32, device=q.device) if vdim > 64 else None
        self._check(self.lib.sb_mlstm_scan(_code(q.dtype), _ptr(q), _ptr(k), _ptr(v), _ptr(g), ld, _ptr(z), z.stride(0), int(i_col),
                                           int(f_col), _ptr(i_bias), _ptr(f_bias), float(cap), _ptr(norm), float(eps), float(q_scale),
                                           float(out_scale), _ptr(state), state.stride(0), self._batch(ctx), heads, dim, vdim,
                                           _ptr(y), y.stride(0), _ptr(raw), self._stream()), "mlstm_scan")
        if raw is not None:
            self.launches += 1   # the norm and the gate
        return y

    def gla_scan(self, ctx, q, k, v, g, z, bias, norm, eps, tau, q_scale, state, heads, dim, vdim):
        """The gated linear recurrence over every sequence's rows, from and back into ``state`` [slots, heads * dim * vdim];
        q, k [rows, heads * dim] and v, g [rows, heads * vdim] may be views of the same wider rows; z [rows, heads * dim] is
        32-bit.  Returns RMSNorm_head(o) * norm * silu(g), [rows, heads * vdim]."""
        rows = q.shape[0]
        ld = q.stride(0)
        for t, w in ((q, heads * dim), (k, heads * dim), (v, heads * vdim), (g, heads * vdim)):
            if tuple(t.shape) != (rows, w) or t.stride(1) != 1 or t.stride(0) != ld or t.dtype != q.dtype:
                raise KernelError("gla_scan: q, k, v, g are views of rows with one stride, in the run's dtype")
        for t in (z, bias, norm, state):
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise KernelError("gla_scan: decay inputs, norm weight and state are 32-bit and contiguous")
        if tuple(z.shape) != (rows, heads * dim) or state.shape[1] != heads * dim * vdim or norm.numel() != vdim:
            raise KernelError("gla_scan: sizes do not fit")
        y = torch.empty((rows, heads * vdim), dtype=q.dtype, device=q.device)
        # heads of more than 64 value channels: their columns are shared out over blocks, which leave raw outputs here
        raw = torch.empty((rows, heads * vdim), dtype=torch.float32, device=q.device) if vdim > 64 else None
        self._check(self.lib.sb_gla_scan(_code(q.dtype), _ptr(q), _ptr(k), _ptr(v), _ptr(g), ld, _ptr(z), _ptr(bias), _ptr(norm),
                                         float(eps), float(tau), float(q_scale), _ptr(state), state.stride(0), self._batch(ctx),
                                         heads, dim, vdim, _ptr(y), _ptr(raw), self._stream()), "gla_scan")
        if raw is not None:
            self.launches += 1   # the norm and the gate
        return y

    def moe_route(self, h, router, correction, top, scale, bias=None, over_chosen=False):
        """(chosen int32 [rows, top], weight 32-bit [rows, top]) of softmax(h router^T + bias) (32-bit): the ``top`` largest
        of score + correction, weighted by their scores over the chosen scores' sum, times ``scale``.  ``over_chosen``:
        the ``top`` largest logits (+ correction) instead, weighted by the softmax over the chosen logits alone.
        ``correction`` and ``bias`` may be None."""
        rows, width = h.shape
        n_out = router.shape[0]
        for extra in (correction, bias):
            if extra is not None and (extra.dtype != torch.float32 or extra.numel() != n_out or not extra.is_contiguous()):
                raise KernelError(f"moe_route: correction and bias are {n_out} 32-bit numbers")
        if (router.dtype != torch.float32 or router.shape[1] != width or not h.is_contiguous()
                or not router.is_contiguous() or n_out > 1024 or top > 32):
            raise KernelError("moe_route: a 32-bit router of up to 1024 outputs, up to 32 choices")
        chosen = torch.empty((rows, top), dtype=torch.int32, device=h.device)
        weight = torch.empty((rows, top), dtype=torch.float32, device=h.device)
        logits = torch.empty((rows, n_out), dtype=torch.float32, device=h.device)
        self._check(self.lib.sb_moe_route(_code(h.dtype), _ptr(h), _ptr(router), _ptr(correction), _ptr(bias), int(bool(over_chosen)),
                                          _ptr(logits), _ptr(chosen), _ptr(weight), rows, width, n_out, int(top), float(scale),
                                          self._stream()), "moe_route")
        self.launches += 1   # logits, then the choice
        return chosen, weight

    MOE_PAIRS_MAX = int(os.environ.get("STARTER_B200_MOE_PAIRS_MAX", 64))   # pairs up to which every pair streams its expert

    def moe_experts(self, h, chosen, weight, w_gate_up, w_down, n_experts, alpha, limit, base):
        """base + sum_k weight[:, k] * expert_chosen[:, k](h): experts are gated feed-forwards (the clamped activation with
        its sigmoid factor ``alpha`` and ``limit``, or silu(gate) * up when ``alpha`` is None) with stacked
        matrices w_gate_up [experts, 2 ff, width] (gate over up) and w_down [experts, width, ff]; a choice >= n_experts
        is an identity output and adds weight * h.  A few pairs: each pair streams its expert's matrices (this library's
        kernels).  Many pairs in bfloat16: the pairs are put in the order of their experts on the device and each matrix
        takes one grouped product of the vendor's library, as the plain products of a prompt do."""
        rows, width = h.shape
        top = chosen.shape[1]
        pairs = rows * top
        dt = _code(h.dtype)
        down = slot_of_pair = None
        if n_experts > 0:
            ff = w_down.shape[2]
            if (tuple(w_gate_up.shape) != (n_experts, 2 * ff, width) or tuple(w_down.shape) != (n_experts, width, ff)
                    or not w_gate_up.is_contiguous() or not w_down.is_contiguous() or w_gate_up.dtype != h.dtype):
                raise KernelError("moe_experts: stacked matrices [experts, 2 ff, width] and [experts, width, ff] in the run's dtype")
            if (h.dtype == torch.bfloat16 and pairs > self.MOE_PAIRS_MAX and width % 8 == 0 and ff % 8 == 0
                    and hasattr(torch, "_grouped_mm")):
                ends = torch.empty(n_experts, dtype=torch.int32, device=h.device)
                slot_of_pair = torch.empty(pairs, dtype=torch.int32, device=h.device)
                pair_of_slot = torch.empty(pairs, dtype=torch.int32, device=h.device)
                self._check(self.lib.sb_moe_sort(_ptr(chosen), pairs, n_experts, _ptr(ends), _ptr(slot_of_pair), _ptr(pair_of_slot),
                                                 self._stream()), "moe_sort")
                xs = torch.zeros((pairs, width), dtype=h.dtype, device=h.device)
                self._check(self.lib.sb_moe_gather(dt, _ptr(h), _ptr(pair_of_slot), _ptr(ends), n_experts, pairs, top, width,
                                                   _ptr(xs), self._stream()), "moe_gather")
                gu = torch._grouped_mm(xs, w_gate_up.transpose(1, 2), offs=ends)
                act = self.swiglu(gu) if alpha is None else self.gated_clamp(gu, alpha, limit)
                down = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)
            else:
                act = torch.empty((pairs, ff), dtype=h.dtype, device=h.device)
                down = torch.empty((pairs, width), dtype=h.dtype, device=h.device)
                self._check(self.lib.sb_moe_pairs(dt, _ptr(h), _ptr(chosen), _ptr(w_gate_up), _ptr(w_down), _ptr(act), _ptr(down),
                                                  pairs, top, n_experts, width, ff, float(alpha or 0.0), float(limit or 0.0),
                                                  int(alpha is None), self._stream()),
                            "moe_pairs")
                self.launches += 1
        y = torch.empty_like(h)
        self._check(self.lib.sb_moe_combine(dt, _ptr(h), _ptr(down), _ptr(base), _ptr(chosen), _ptr(weight), _ptr(slot_of_pair),
                                            _ptr(y), rows, top, n_experts, width, self._stream()), "moe_combine")
        return y

    # ---- a layer whose branches read the 32-bit residual itself: position vector, short convolution, branch norm ----

    def embed_sinusoid(self, ctx, tokens, table, freqs):
        """32-bit rows table[token] + position vector: column 2i takes sin(position * freqs[i]), column 2i + 1 the cosine;
        the angle is formed and turned in 32-bit in the kernel."""
        rows, width = tokens.shape[0], table.shape[1]
        if freqs.dtype != torch.float32 or freqs.numel() * 2 < width or not table.is_contiguous():
            raise KernelError(f"embed_sinusoid: {(width + 1) // 2} 32-bit frequencies for rows of {width} columns")
        out = torch.empty((rows, width), dtype=torch.float32, device=table.device)
        self._check(self.lib.sb_embed_sinusoid(_code(table.dtype), _ptr(tokens), _ptr(table), _ptr(freqs), _ptr(out), self._batch(ctx),
                                               width, table.shape[0], _ptr(ctx.status), self._stream()), "embed_sinusoid")
        return out

    def cast_rows(self, x, dtype):
        """The 32-bit rows rounded to ``dtype`` (what a branch reads when nothing stands before it)."""
        if x.dtype == dtype:
            return x
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("cast_rows: contiguous 32-bit rows")
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        self._check(self.lib.sb_causal_conv(_code(dtype), _ptr(x), None, None, 0, SbBatch(None, None, None, None, 0, x.shape[0], 0, 0),
                                            x.shape[1], 0, _ptr(out), self._stream()), "cast_rows")
        return out

    def causal_conv(self, ctx, x, weight, state, out_dtype):
        """x_t + sum_j weight[:, j] * x_(t - taps + 1 + j) per sequence and column, 32-bit sum, rounded to ``out_dtype``;
        ``state`` [slots, taps - 1, width] (32-bit) holds each sequence's last inputs and is brought up to date."""
        rows, width = x.shape
        taps = weight.shape[1]
        if (x.dtype != torch.float32 or weight.dtype != torch.float32 or tuple(weight.shape) != (width, taps) or not x.is_contiguous()
                or not weight.is_contiguous()):
            raise KernelError("causal_conv: 32-bit rows and a 32-bit [width, taps] weight")
        if taps > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, width)
                         or not state.is_contiguous()):
            raise KernelError(f"causal_conv: the state is [slots, {taps - 1}, {width}] 32-bit numbers")
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
        self._check(self.lib.sb_causal_conv(_code(out_dtype), _ptr(x), _ptr(weight), _ptr(state) if taps > 1 else None,
                                            (taps - 1) * width, self._batch(ctx), width, taps, _ptr(out), self._stream()),
                    "causal_conv")
        if taps > 1:
            self.launches += 1   # the state's kernel
        return out

    def branch_norm_add(self, x, y, weight, scale, eps, out_dtype, next_norm=None):
        """x += y / sqrt(mean(y^2) + eps) * weight (* scale), in place and 32-bit; returns the new x rounded to
        ``out_dtype`` (x itself when it has that type), or None when ``out_dtype`` is None.  ``next_norm`` = (weight, eps)
        of the RMS norm that the next branch takes of the residual: the kernel then returns that norm of the new x in
        y's type instead (one pass over the row for the sum, the norm and the rounding)."""
        rows, width = x.shape
        if next_norm is not None:
            next_w, next_eps = next_norm
            if next_w.dtype != torch.float32 or next_w.numel() != width or not next_w.is_contiguous():
                raise KernelError("branch_norm_add: the next norm's weight is 32-bit, one per column")
            if (x.dtype != torch.float32 or tuple(y.shape) != (rows, width) or not x.is_contiguous() or not y.is_contiguous()
                    or weight.dtype != torch.float32 or weight.numel() != width or scale is not None):
                raise KernelError("branch_norm_add: a contiguous 32-bit residual, a branch output of its shape, 32-bit weights")
            normed = torch.empty((rows, width), dtype=y.dtype, device=x.device)
            self._check(self.lib.sb_branch_norm_add(_code(y.dtype), _ptr(x), _ptr(y), _ptr(weight), None, None, rows, width, float(eps),
                                                    _ptr(next_w), float(next_eps), _ptr(normed), self._stream()), "branch_norm_add")
            return normed
        if (x.dtype != torch.float32 or tuple(y.shape) != (rows, width) or not x.is_contiguous() or not y.is_contiguous()
                or weight.dtype != torch.float32 or weight.numel() != width or (scale is not None and (scale.dtype != torch.float32
                                                                                                    or scale.numel() != width))):
            raise KernelError("branch_norm_add: a contiguous 32-bit residual, a branch output of its shape, 32-bit weights")
        rounded = None
        if out_dtype is not None and out_dtype != torch.float32:
            if out_dtype != y.dtype:
                raise KernelError("branch_norm_add: the rounded copy has the branch output's type")
            rounded = torch.empty((rows, width), dtype=out_dtype, device=x.device)
        self._check(self.lib.sb_branch_norm_add(_code(y.dtype), _ptr(x), _ptr(y), _ptr(weight), _ptr(scale), _ptr(rounded), rows, width,
                                                float(eps), None, 0.0, None, self._stream()), "branch_norm_add")
        if out_dtype is None:
            return None
        return x if rounded is None else rounded

    def xielu(self, z, a_pos, a_neg):
        """a_pos z^2 + z / 2 for z > 0, a_neg (exp(z) - 1 - z) + z / 2 otherwise, element by element."""
        if not z.is_contiguous():
            raise KernelError("xielu: a contiguous tensor")
        out = torch.empty_like(z)
        self._check(self.lib.sb_xielu(_code(z.dtype), _ptr(z), _ptr(out), z.numel(), float(a_pos), float(a_neg), self._stream()),
                    "xielu")
        return out

    def linear_xielu(self, h, w_up, a_pos, a_neg):
        """xielu(h @ w_up^T).  For the few rows of a decode step the activation sits in the product's epilogue, as SwiGLU
        does in ``linear_swiglu``."""
        M, K = h.shape
        if h.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and K % 8 == 0 and M <= self.SKINNY_MAX_ROWS:
            return self._skinny(h, w_up, w_up.shape[0], False, False, unary=(a_pos, a_neg))
        return self.xielu(self.linear(h, w_up), a_pos, a_neg)

    def qk_norm_store(self, ctx, qkv, layer_cache, n_heads, q_norm, k_norm, eps):
        """From rows [q | k | v]: the query part divided by the root mean square of the WHOLE part (all heads at once) times
        ``q_norm``, the key part likewise with ``k_norm`` (None: nothing is normed); keys and values go to the layer's
        cache, the queries come back as [rows, heads, key width]."""
        g = layer_cache.group
        G, D, V = g.request.num_kv_heads, g.request.head_dim, g.v_dim
        rows = qkv.shape[0]
        nq = n_heads * D
        if (qkv.shape[1] != nq + G * (D + V) or not qkv.is_contiguous() or qkv.dtype != layer_cache.k.dtype or g.v_heads != G):
            raise KernelError(f"qk_norm_store: rows of {nq} + {G * D} + {G * V} columns in the cache's type, not {tuple(qkv.shape)}")
        for w, n in ((q_norm, nq), (k_norm, G * D)):
            if w is not None and (w.dtype != torch.float32 or w.numel() != n):
                raise KernelError("qk_norm_store: 32-bit norm weights over the whole query and the whole key part")
        q = torch.empty((rows, n_heads, D), dtype=qkv.dtype, device=qkv.device)
        p = self._flex(layer_cache)
        self._check(self.lib.sb_qk_norm_store(_code(qkv.dtype), _ptr(qkv), _ptr(q), self._batch(ctx), p, n_heads, _ptr(q_norm),
                                              _ptr(k_norm), float(eps), _ptr(ctx.status), self._stream()), "qk_norm_store")
        return q

    def talking_attention(self, ctx, q, layer_cache, n_heads, scale, softcap=None, talk=None, sink=None, window=None, keep_first=0):
        """Causal attention whose capped scores are mixed across heads before the softmax: q [rows, heads, key width] over
        the layer's cache -> [rows, heads * value width].  s_g = softcap * tanh(q_g.k * scale / softcap); t_h = sum_g
        talk[h, g] s_g; a row at position i sees key j <= i when i - j < window or j < keep_first; exp(sink_h) joins the
        softmax's denominator.  Every option is off when None / 0."""
        rows, H, kd = q.shape
        g = layer_cache.group
        if H != n_heads or q.stride(2) != 1 or kd != g.request.head_dim or q.dtype != layer_cache.k.dtype:
            raise KernelError(f"talking_attention: q {tuple(q.shape)} {q.dtype} does not fit the layer's cache")
        if H % g.request.num_kv_heads:
            raise KernelError(f"{H} query heads cannot share {g.request.num_kv_heads} key/value heads evenly")
        for t, n in ((talk, H * H), (sink, H)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
                raise KernelError("talking_attention: a 32-bit [heads, heads] table and 32-bit sinks per head")
        if keep_first and not window:
            raise KernelError("talking_attention: kept first keys go with a window")
        p = self._flex(layer_cache, q, H, scale, g.v_dim, False, sink, None, None, None, window, keep_first, softcap, talk)
        out = torch.empty((rows, H * g.v_dim), dtype=q.dtype, device=q.device)
        mma = self._talk_takes_mma(ctx, q, p)
        n_splits = self.talk_mma_splits(ctx, p, g.table_width) if mma else self.talk_splits(ctx, p, g.table_width)
        partial = None
        if n_splits > 1:
            key = ("talk_partial", q.device, rows, H, n_splits, g.v_dim)
            partial = self._scratch.get(key)
            if partial is None:
                partial = self._scratch[key] = torch.empty(rows * H * n_splits * (g.v_dim + 2), dtype=torch.float32, device=q.device)
        if mma:
            self._check(self.lib.sb_talking_attention_mma(p, self._batch(ctx), _ptr(out), ctx.max_q_len, n_splits, _ptr(partial),
                                                          self._stream()), "talking_attention_mma")
        else:
            self._check(self.lib.sb_talking_attention_general(_code(q.dtype), p, self._batch(ctx), _ptr(out), n_splits, _ptr(partial),
                                                              self._stream()), "talking_attention_general")
        if n_splits > 1:
            self.launches += 1   # the merge of the splits
        return out

    TALK_PROMPT_MIN_ROWS = 4

    def _talk_takes_mma(self, ctx, q, p: SbFlex) -> bool:
        """The tensor-core kernel (16 positions with all their heads per block) takes bfloat16 steps in which a sequence
        brings at least 4 rows, key widths that are multiples of 16, values of 64 or 128 columns, up to 32 heads (16 with
        values of 128 columns) and rows it can fetch 16 bytes at a time; the block-per-row kernel serves everything else
        (decoding, and every 32-bit run)."""
        if not self.flex_tensor_cores or q.dtype != torch.bfloat16 or ctx.max_q_len < self.TALK_PROMPT_MIN_ROWS:
            return False
        smem = self.lib.sb_talking_attention_mma_smem(p.n_heads, p.n_kv_heads, p.k_dim, p.v_dim)
        if smem < 0 or smem > self.MAX_BLOCK_SHARED:
            return False
        return q.stride(0) % 8 == 0 and q.stride(1) % 8 == 0 and q.data_ptr() % 16 == 0 and p.v_row % 8 == 0

    def talk_splits(self, ctx, p: SbFlex, max_pages: int) -> int:
        """Blocks along the keys per row of the block-per-row kernel: enough for two blocks per SM, none with less than
        one turn of 32 keys.  A function of shapes only, so that a captured graph stays valid."""
        reach = max_pages * 64
        if p.window:
            reach = min(reach, p.window + p.keep_first)
        turns = max(1, (min(reach, ctx.kv_bound) + 31) // 32)
        return max(1, min(-(-2 * self.sm_count() // max(1, ctx.n_rows)), turns, 64))

    def talk_mma_splits(self, ctx, p: SbFlex, max_pages: int) -> int:
        """Blocks along the keys per 16 positions of the tensor-core kernel: one block holds an SM (its scores of all heads
        fill the shared memory), so a step of few positions with many keys in reach is cut until there are three blocks per
        SM (measured at 128 blocks of positions: four shares 186 and 388 us where one takes 209 and 706), none with less
        than 128 keys, four at most."""
        reach = max_pages * 64
        if p.window:
            reach = min(reach, p.window + p.keep_first + 16)
        reach = min(reach, ctx.kv_bound)
        blocks = ctx.n_seqs * -(-ctx.max_q_len // 16)
        return max(1, min(-(-3 * self.sm_count() // max(1, blocks)), reach // 128, 4))

    # ---- sampling -----------------------------------------------------------------------

    def argmax(self, logits):
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        key = ("argmax", logits.device, rows)
        buf = self._scratch.get(key)
        if buf is None:
            buf = self._scratch[key] = (torch.empty(rows * 32, dtype=torch.float32, device=logits.device),
                                        torch.empty(rows * 32, dtype=torch.int32, device=logits.device))
        self._check(self.lib.sb_argmax(_ptr(logits), _ptr(out), rows, logits.shape[1], _ptr(buf[0]), _ptr(buf[1]),
                                       self._stream()), "argmax")
        return out

    def sample(self, logits, temperature, top_k, seed, request_ids, steps, advance=False, device_params=None):
        """``device_params``: int32 [4] on the device {temperature's float bits, top_k, seed low, seed high};
        when given, the kernel reads them there as it runs (a captured step then serves every setting)."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        self._check(self.lib.sb_sample(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], float(temperature),
                                       int(top_k), int(seed) & ((1 << 64) - 1), _ptr(request_ids), _ptr(steps),
                                       int(bool(advance)), _ptr(device_params), self._stream()), "sample")
        return out


_OPS = None


def get_ops(verbose: bool = True) -> Ops:
    """The extension's call table.  Raises if there is no CUDA device or the library cannot be built."""
    global _OPS
    if _OPS is None:
        if not torch.cuda.is_available():
            raise BuildError("no CUDA device: this library runs on a B200 only and has no other path")
        _OPS = Ops(load(verbose=verbose))
    return _OPS
