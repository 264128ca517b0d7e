"""ctypes bindings of the CUDA kernels.

Every method takes torch CUDA tensors, launches on torch's current stream and
raises `KernelError` when the entry point refuses its arguments or the launch
fails.  There is no CPU path: without a CUDA device, or without the compiled
library, `get_kernels()` raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_float, c_void_p, c_char_p
from typing import List, Optional

import torch

from . import build

F32, BF16 = 0, 1
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}      # the gate's activation in gated feed-forwards (common.cuh BRAID_ACT_*)


def activation_code(name: str) -> int:
    if name not in ACTIVATIONS:
        raise KernelError(f"unknown activation {name!r}; the kernels have {sorted(ACTIVATIONS)}")
    return ACTIVATIONS[name]


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dt}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def token_tile(rows: int) -> int:
    """The token tile (UMMA N) of the tensor-core product for a step of `rows` tokens: the
    smallest of 16, 32, 64, 128, 256 that holds them, 256 beyond.  The one place the ladder
    is written: the kernel is told the tile, and whoever sizes work by it asks here."""
    for t in (16, 32, 64, 128):
        if rows <= t:
            return t
    return 256


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the SwiGLU epilogue: blocks of 32 rows, each the gate rows
    [16t, 16t+16) followed by the up rows [16t, 16t+16); rows past the true size are zero."""
    inter, k = gate.shape
    blocks = -(-inter // 16)
    g = torch.zeros((blocks * 16, k), dtype=gate.dtype, device=gate.device)
    u = torch.zeros_like(g)
    g[:inter] = gate
    u[:inter] = up
    return torch.cat([g.view(blocks, 16, k), u.view(blocks, 16, k)], dim=1).reshape(blocks * 32, k).contiguous()


PAIR_TOKEN_TILE = 256        # the token tile of the kernel that runs on pairs of SMs
# Tokens a chunk of a long prompt's recurrence (csrc/scan.cu): 128 for sequences of 1,024 tokens and more, 64 below
# (2,048 tokens, 8 heads of 128 x 256: 0.42 / 0.32 / 0.29 / 0.30 ms with chunks of 32 / 64 / 128 / 256); steps whose
# longest sequence brings less than two chunks walk in one pass.  BRAIDINFER_SCAN_CHUNK names one length for all
# (0: never in chunks), for measurements.
SCAN_CHUNK = int(os.environ["BRAIDINFER_SCAN_CHUNK"]) if os.environ.get("BRAIDINFER_SCAN_CHUNK") else None


class RowScale:
    """A row scale still to be applied: an RMSNorm whose rows were left unscaled (csrc/rowscale.cuh).
    `shares` [n, stride >= rows] float32 holds each row's sum of squares in n shares, as the kernel that
    wrote the rows left them; the scale of row r is rsqrt(sum over shares[:, r] / width + eps).  The
    product that reads the unscaled rows applies the scale to its own results (`in_scale`)."""

    def __init__(self, shares: torch.Tensor, width: int, eps: float) -> None:
        self.shares, self.width, self.eps = shares, int(width), float(eps)

    def args(self):
        return (self.shares.data_ptr(), self.shares.shape[0], self.shares.stride(0), float(self.width), self.eps)

    def values(self) -> torch.Tensor:
        """The scales themselves (for tests and for parts written in torch)."""
        return torch.rsqrt(self.shares.sum(0) / self.width + self.eps)


_NO_SCALE = (None, 0, 0, 0.0, 0.0)
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)      # torch's own quick way to the stream handle


def _scale_args(scale: Optional["RowScale"]):
    return scale.args() if scale is not None else _NO_SCALE


class PartialProduct:
    """Partial products of a stream-k GEMM waiting in the workspace to be added up."""

    def __init__(self, workspace: torch.Tensor, plan, n_rows: int, w_rows: int,
                 rs_rows: Optional[torch.Tensor] = None) -> None:
        self.workspace, self.plan, self.n_rows, self.w_rows = workspace, plan, n_rows, w_rows
        # the scale of every row that the product's input still wants (float32 [n_rows], written by the
        # product's kernel from the RowScale it was given): the adding-up has to apply it
        self.rs_rows = rs_rows


class Kernels:
    """The loaded kernel library.  One instance per process (`get_kernels`)."""

    def __init__(self, verbose: bool = True) -> None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: braidinfer_b200 runs on an NVIDIA B200 (sm_100a) only "
                              "and has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
        path = build.core_library(verbose=verbose)
        self.lib = ctypes.CDLL(str(path))
        self.path = str(path)
        self.launches = 0          # kernels launched through this object (for measurements)
        self._declare()
        self._device_index = torch.cuda.current_device()
        self._error_flag = torch.zeros(8, dtype=torch.int32, device="cuda")
        self._tc_workspace: Optional[torch.Tensor] = None
        self._attn_libs = {}
        self._part_libs = {}
        self.pending_partial = None     # the open PartialProduct, if any (it owns the GEMM workspace)
        self.workspace_generation = 0   # grows when a scratch buffer moves (captured graphs are stale then)
        self._attn_partial: Optional[torch.Tensor] = None
        self._verbose = verbose

    # ------------------------------------------------------------------ plumbing
    def _declare(self) -> None:
        L = self.lib
        L.braid_last_error.restype = c_char_p
        L.braid_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        L.braid_embed_pos.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                      c_int, c_void_p, c_void_p]
        L.braid_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_float,
                                    c_void_p]
        L.braid_head_prep_kv.argtypes = [c_void_p, c_longlong, c_int] + [c_void_p] * 5 + [c_int] * 10 + \
                                        [c_float, c_float, c_int, c_void_p, c_void_p]
        L.braid_head_gate.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p] + [c_int] * 5 + [c_void_p]
        L.braid_glu_clamp.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p]
        L.braid_silu_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.braid_act_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        L.braid_head_norm_rope_kv.argtypes = [c_void_p, c_longlong, c_int] + [c_void_p] * 7 + [c_int] * 10 + \
                                             [c_float, c_float, c_void_p, c_void_p]
        L.braid_act_mul_gather.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                                           c_int, c_int, c_int, c_int, c_void_p]
        L.braid_rmsnorm_add.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p]
        L.braid_residual_add.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
        L.braid_rope_kv_write.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p]
        L.braid_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
        L.braid_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        L.braid_gather_i32.restype = c_int
        L.braid_attn_simple.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_int, c_float, c_float, c_void_p, c_void_p, c_longlong, c_int, c_void_p,
                                        c_int, c_void_p, c_void_p]
        L.braid_head_mix.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p] + \
                                    [c_int] * 5 + [c_void_p]
        L.braid_bias_xielu.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_longlong] + [c_int] * 4 + \
                                      [c_void_p]
        L.braid_gemm_simt.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p]
        scale = [c_void_p, c_int, c_longlong, c_float, c_float]        # RowScale.args()
        L.braid_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                    c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
                                    c_void_p] + scale + [c_void_p, c_void_p, c_void_p]
        L.braid_streamk_reduce_prep.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                c_longlong, c_int, c_void_p]
        L.braid_gemm_tc2.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_longlong, c_longlong, c_longlong, c_int, c_void_p, c_void_p]
        L.braid_streamk_reduce.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong,
                                           c_int, c_int, c_void_p, c_void_p]
        L.braid_streamk_reduce_norm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                c_void_p, c_int, c_int, c_float, c_void_p]
        L.braid_streamk_reduce_rope_kv.argtypes = [c_void_p] * 8 + [c_int] * 9 + [c_void_p, c_void_p, c_void_p]
        L.braid_gemm_tc_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int]
        L.braid_gemm_tc_workspace_bytes.restype = c_longlong
        L.braid_logit_hash.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p]
        L.braid_logit_hash.restype = c_int
        L.braid_argmax.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p]
        L.braid_sample.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 12 + \
                                  [c_void_p, c_void_p]
        L.braid_dyt.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                c_float, c_void_p]
        L.braid_softcap.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        L.braid_concat2.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        for name in ("braid_dyt", "braid_softcap", "braid_concat2", "braid_head_mix", "braid_bias_xielu"):
            getattr(L, name).restype = c_int
        for name in ("braid_embed", "braid_embed_pos", "braid_head_prep_kv", "braid_head_gate", "braid_glu_clamp", "braid_rmsnorm", "braid_silu_mul", "braid_act_mul", "braid_head_norm_rope_kv",
                     "braid_act_mul_gather", "braid_rmsnorm_add", "braid_residual_add",
                     "braid_rope_kv_write", "braid_cast", "braid_attn_simple", "braid_gemm_simt",
                     "braid_gemm_tc", "braid_gemm_tc2", "braid_argmax", "braid_sample", "braid_streamk_reduce",
                     "braid_streamk_reduce_norm", "braid_streamk_reduce_rope_kv", "braid_streamk_reduce_prep",
                     "braid_streamk_reduce_prep_cols"):
            getattr(L, name).restype = c_int

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            msg = self.lib.braid_last_error().decode(errors="replace")
            raise KernelError(f"{what}: {msg} (code {rc})")

    def _stream(self):
        """The current stream's handle (inside a graph capture: the capturing stream).  Asked for at every
        launch, so through the quick route where this torch has it."""
        if _RAW_STREAM is not None:
            return _RAW_STREAM(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def check_device_errors(self) -> None:
        """Read the flags that kernels raise (a cache write outside its pages, a
        tensor-core kernel whose bounded wait ran out, NaN logits) and raise on any.
        It synchronises the stream, so the step calls it where it reads results."""
        flags = self._error_flag.tolist()
        if any(flags):
            self._error_flag.zero_()
            names = ["cache write outside the sequence's pages", "tensor-core GEMM wait ran out",
                     "NaN among the logits",
                     "tcgen05 attention gave up (a wait ran out, a visible position had no page, or its shared "
                     "memory was not 1024-byte aligned)",
                     "attention met a visible position whose page is absent or outside the cache (it read page 0 "
                     "instead; the result is wrong)",
                     "a token stands at a position past the model's table of positions"]
            raise KernelError("device error: " + "; ".join(n for n, f in zip(names, flags) if f))

    # ------------------------------------------------------------------ row-wise kernels
    def logit_hash(self, logits: torch.Tensor) -> List[int]:
        """One 64-bit hash a row of float32 logits (FNV-1a over the elements' 32-bit patterns, the hash the
        reference logs under BRAIDINFER_LOGIT_TRACE): equal logits, equal hash, so the first step at which
        two runs part is found by comparing two short text files.  Synchronises."""
        if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
            raise KernelError("logit_hash wants float32 rows [n, vocab] with contiguous elements")
        n, vocab = logits.shape
        out = torch.empty(max(n, 1), dtype=torch.int64, device=logits.device)
        self.launches += 1
        self._check(self.lib.braid_logit_hash(logits.data_ptr(), logits.stride(0), n, vocab, out.data_ptr(),
                                              self._stream()), "logit_hash")
        return [v & 0xFFFFFFFFFFFFFFFF for v in out[:n].tolist()]

    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
              pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> None:
        """out[t] = table[ids[t]] * scale, float32; with `pos_table` ([positions, hidden], the table's element type)
        plus pos_table[positions[t]], unscaled.  A position past the table raises the cache flag and adds nothing."""
        n, hidden = out.shape
        self.launches += 1
        if pos_table is not None:
            if pos_table.dtype != table.dtype or pos_table.shape[1] != hidden or not pos_table.is_contiguous() or positions is None:
                raise KernelError("embed: the table of positions has the token table's element type and width, and needs positions")
            self._check(self.lib.braid_embed_pos(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                                                 n, hidden, table.shape[0], float(scale), pos_table.data_ptr(),
                                                 positions.data_ptr(), pos_table.shape[0], self._error_flag.data_ptr() + 20,
                                                 self._stream()), "embed")
            return
        self._check(self.lib.braid_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                                         n, hidden, table.shape[0], float(scale), self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float,
                row_index: Optional[torch.Tensor] = None, w_offset: float = 0.0) -> None:
        """out = x / sqrt(mean(x^2) + eps) * (w + w_offset), row by row (w_offset 1: zero-centred weights)."""
        rows, width = out.shape
        if x.dtype != torch.float32:
            raise KernelError("rmsnorm reads the float32 residual stream")
        self.launches += 1
        self._check(self.lib.braid_rmsnorm(x.data_ptr(), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                                           dtype_code(out.dtype), _ptr(row_index), rows, width, float(eps),
                                           float(w_offset), self._stream()), "rmsnorm")

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor) -> None:
        self.act_mul(gu, out, "silu")

    def act_mul(self, gu: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
        """out = act(gu[:, :I]) * gu[:, I:], I = out's width."""
        rows, inter = out.shape
        self.launches += 1
        self._check(self.lib.braid_act_mul(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), rows, inter,
                                           activation_code(activation), self._stream()), "act_mul")

    def head_norm_rope_kv(self, qk: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                          inv_freq: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                          page_table: Optional[torch.Tensor], cache: Optional[torch.Tensor], nqh: int, nkh: int, hd: int,
                          rope_dim: int, adjacent: bool, value_is_key: bool, page_size: int, eps: float,
                          amp: float = 1.0) -> None:
        """Rows of stacked heads [rows, >= (nqh + nkh (+ nkh)) * hd]: every query and key head is RMS-normed over
        the head with q_w / k_w ([hd], shared by the heads; None: no norm), rotated (sine and cosine times `amp`)
        and written back; keys also go into the cache's key plane, and the value plane takes the value heads, or,
        with `value_is_key`, the key heads as they came in (before norm and rotation)."""
        for w in (q_w, k_w):
            if w is not None and (w.dtype != qk.dtype or w.numel() != hd):
                raise KernelError(f"head_norm_rope_kv: a norm weight must hold {hd} numbers of the rows' element type")
        if cache is not None and cache.dtype != qk.dtype:
            raise KernelError("head_norm_rope_kv: rows and cache must have one element type")
        if qk.stride(1) != 1 or qk.shape[1] < (nqh + (nkh if value_is_key else 2 * nkh)) * hd:
            raise KernelError("head_norm_rope_kv: the rows do not hold the heads")
        cols = page_table.shape[1] if page_table is not None else 0
        self.launches += 1
        self._check(self.lib.braid_head_norm_rope_kv(
            qk.data_ptr(), qk.stride(0), dtype_code(qk.dtype), _ptr(q_w), _ptr(k_w), inv_freq.data_ptr(),
            positions.data_ptr(), token_seq.data_ptr(), _ptr(page_table), _ptr(cache), qk.shape[0], nqh, nkh, hd,
            rope_dim, int(adjacent), int(value_is_key), page_size, cols, cache.shape[0] if cache is not None else 0,
            float(eps), float(amp), self._error_flag.data_ptr(), self._stream()), "head_norm_rope_kv")

    def act_mul_gather(self, gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int, out: torch.Tensor,
                       activation: str) -> None:
        """out[r, j] = act(gate[r, j]) * table[ids[r], col0 + j]."""
        rows, dim = out.shape
        if not (gate.dtype == table.dtype == out.dtype) or not out.is_contiguous() or gate.stride(1) != 1 \
                or table.stride(1) != 1 or col0 + dim > table.shape[1] or gate.shape[1] < dim:
            raise KernelError("act_mul_gather: gate, table and out of one element type; the table must hold the columns")
        self.launches += 1
        self._check(self.lib.braid_act_mul_gather(gate.data_ptr(), gate.stride(0), table.data_ptr(), table.stride(0),
                                                  ids.data_ptr(), table.shape[0], int(col0), out.data_ptr(),
                                                  dtype_code(out.dtype), rows, dim, activation_code(activation),
                                                  self._stream()), "act_mul_gather")

    def rmsnorm_add(self, h: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> None:
        """h += y / sqrt(mean(y^2) + eps) * (w + w_offset), row by row; h and y float32 [rows, width], contiguous."""
        if h.dtype != torch.float32 or y.dtype != torch.float32 or h.shape != y.shape or not h.is_contiguous() \
                or not y.is_contiguous() or w.numel() != h.shape[1]:
            raise KernelError("rmsnorm_add: h and y are contiguous float32 of one shape, w one number a column")
        self.launches += 1
        self._check(self.lib.braid_rmsnorm_add(h.data_ptr(), y.data_ptr(), w.data_ptr(), dtype_code(w.dtype), h.shape[0],
                                               h.shape[1], float(eps), float(w_offset), self._stream()), "rmsnorm_add")

    def head_prep_kv(self, src: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                     page_table: Optional[torch.Tensor], cache: Optional[torch.Tensor], nqh: int, nkh: int, dk: int, dv: int,
                     hd: int, unit: bool, eps: float, temp_coef: float = 0.0, temp_every: int = 0) -> None:
        """Rows of stacked heads without rotation (nqh query heads of dk, nkh key heads of dk, nkh value heads of dv):
        with `unit` queries and keys are divided by their root mean square over the head; queries are multiplied by
        1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: not); queries go to q_out [rows, nqh * hd],
        keys and values into the cache's planes, each padded with zeros up to hd."""
        if src.stride(1) != 1 or src.shape[1] < nqh * dk + nkh * (dk + dv) or q_out.dtype != src.dtype \
                or tuple(q_out.shape) != (src.shape[0], nqh * hd) or not q_out.is_contiguous():
            raise KernelError("head_prep_kv: the rows do not hold the heads, or q_out is not [rows, heads * padded size]")
        if cache is not None and (cache.dtype != src.dtype or cache.shape[-1] != hd or cache.shape[1] != 2 or cache.shape[2] != nkh):
            raise KernelError("head_prep_kv: the cache is [pages, 2, kv_heads, page, padded size] of the rows' element type")
        self.launches += 1
        self._check(self.lib.braid_head_prep_kv(
            src.data_ptr(), src.stride(0), dtype_code(src.dtype), q_out.data_ptr(), positions.data_ptr(), token_seq.data_ptr(),
            _ptr(page_table), _ptr(cache), src.shape[0], nqh, nkh, dk, dv, hd, int(unit),
            cache.shape[3] if cache is not None else build.page_size(), page_table.shape[1] if page_table is not None else 0,
            cache.shape[0] if cache is not None else 0, float(eps), float(temp_coef), int(temp_every),
            self._error_flag.data_ptr(), self._stream()), "head_prep_kv")

    def head_gate(self, x: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, heads: int, hd: int, dv: int) -> None:
        """out[r, h * dv + c] = x[r, h * hd + c] * sigmoid(gate[r, h]), c < dv (gate None: the copy alone)."""
        rows = out.shape[0]
        if x.stride(1) != 1 or not out.is_contiguous() or out.shape[1] != heads * dv or x.dtype != out.dtype \
                or (gate is not None and (gate.dtype != x.dtype or gate.stride(1) != 1 or gate.shape[1] < heads)):
            raise KernelError("head_gate: x, gate and out of one element type; out contiguous [rows, heads * dv]")
        self.launches += 1
        self._check(self.lib.braid_head_gate(x.data_ptr(), x.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                             out.data_ptr(), dtype_code(out.dtype), rows, heads, hd, dv, self._stream()),
                    "head_gate")

    def glu_clamp(self, gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
        """out = g * sigmoid(alpha * g) * (u + 1), g = min(gu[:, :I], limit), u = clamp(gu[:, I:], -limit, limit)."""
        rows, inter = out.shape
        if not gu.is_contiguous() or not out.is_contiguous() or gu.shape[1] != 2 * inter or gu.dtype != out.dtype:
            raise KernelError("glu_clamp: gu contiguous [rows, 2 I], out contiguous [rows, I], one element type")
        self.launches += 1
        self._check(self.lib.braid_glu_clamp(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), rows, inter, float(limit),
                                             float(alpha), self._stream()), "glu_clamp")

    def residual_add(self, h: torch.Tensor, delta: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_residual_add(h.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype),
                                                h.numel(), self._stream()), "residual_add")

    def cast(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_cast(src.data_ptr(), dtype_code(src.dtype), dst.data_ptr(),
                                        dtype_code(dst.dtype), src.numel(), self._stream()), "cast")

    def gather_i32(self, src: torch.Tensor, index: torch.Tensor, dst: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_gather_i32(src.data_ptr(), index.data_ptr(), dst.data_ptr(), index.numel(),
                                              self._stream()), "gather_i32")

    def rope_kv_write(self, qkv: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor,
                      token_seq: torch.Tensor, page_table: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                      nqh: int, nkh: int, hd: int, rope_dim: int, adjacent: bool, page_size: int) -> None:
        rows = qkv.shape[0]
        cols = page_table.shape[1] if page_table is not None else 0
        num_pages = cache.shape[0] if cache is not None else 0
        self.launches += 1
        self._check(self.lib.braid_rope_kv_write(
            qkv.data_ptr(), dtype_code(qkv.dtype), inv_freq.data_ptr(), positions.data_ptr(), token_seq.data_ptr(),
            _ptr(page_table), _ptr(cache), rows, nqh, nkh, hd, rope_dim, int(adjacent), page_size, cols, num_pages,
            self._error_flag.data_ptr(), self._stream()), "rope_kv_write")

    def attn_simple(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, nqh: int, nkh: int, hd: int,
                    page_size: int, window: Optional[int], scale: float, sink: Optional[float] = None,
                    out_scale: float = 1.0, head_sinks: Optional[torch.Tensor] = None,
                    head_gate: Optional[torch.Tensor] = None, keep_first: int = 0,
                    head_scale: Optional[torch.Tensor] = None, value_heads: int = 1) -> None:
        """q: [rows, >= nqh*hd] (a view of the qkv rows is fine), out: [rows, nqh*hd].  `keep_first`: with a window,
        a sequence's first positions stay visible; `head_scale` (float32 [nqh]): a factor a head on the scores;
        `value_heads` = nkh: every query head reads the values of every kv head, out is [rows, nqh*nkh*hd] with
        the result of (head h, value head c) at virtual head h*nkh + c (see `head_mix`).  `sink`: the score of an
        attention sink, one more term of the softmax's denominator that has no value (None: no sink);
        `head_sinks` (float32 [nqh]): a sink score a head instead; `out_scale`: a constant factor on the result;
        `head_gate` ([rows, >= nqh] of the rows' type, a view is fine): head h's result times sigmoid(head_gate[row, h])."""
        rows = out.shape[0]
        self._check_head_extras(head_sinks, head_gate, nqh, out.dtype, head_scale)
        if out.shape[1] < nqh * value_heads * hd:
            raise KernelError("attn_simple: the result's rows do not hold the heads")
        self.launches += 1
        self._check(self.lib.braid_attn_simple(
            q.data_ptr(), out.data_ptr(), dtype_code(out.dtype), cache.data_ptr(), page_table.data_ptr(),
            positions.data_ptr(), token_seq.data_ptr(), q.stride(0), out.stride(0), rows, nqh, nkh, hd,
            page_size, page_table.shape[1], cache.shape[0], int(window or 0), float(scale),
            int(sink is not None), float(sink or 0.0), float(out_scale), _ptr(head_sinks), _ptr(head_gate),
            head_gate.stride(0) if head_gate is not None else 0, int(keep_first or 0), _ptr(head_scale), int(value_heads),
            self._error_flag.data_ptr() + 16, self._stream()),
            "attn_simple")

    def head_mix(self, src: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, token_seq: Optional[torch.Tensor],
                 heads: int, kv_heads: int, hd: int, vd: int) -> None:
        """out[row, h, :vd] = sum_g talk[h, g] * src[row, g * kv_heads + kv(h), :vd]: src [rows, heads * kv_heads * hd] is what
        attention leaves when every head reads the values of every kv head, talk [heads, heads] mixes the heads'
        probabilities after the softmax, out [rows, heads * vd].  float32 sums; rows of padding come out zero."""
        rows = src.shape[0]
        if src.stride(1) != 1 or out.stride(1) != 1 or src.shape[1] < heads * kv_heads * hd or out.shape[1] < heads * vd \
                or src.dtype != out.dtype or tuple(talk.shape) != (heads, heads) or not talk.is_contiguous():
            raise KernelError("head_mix: src [rows, heads * kv_heads * hd], talk contiguous [heads, heads], out [rows, heads * vd]")
        self.launches += 1
        self._check(self.lib.braid_head_mix(src.data_ptr(), src.stride(0), talk.data_ptr(), dtype_code(talk.dtype),
                                            out.data_ptr(), out.stride(0), dtype_code(out.dtype), _ptr(token_seq), rows, heads,
                                            kv_heads, hd, vd, self._stream()), "head_mix")

    def bias_xielu(self, z: torch.Tensor, bias: torch.Tensor, pq: torch.Tensor, out: torch.Tensor, n: int) -> None:
        """out[:, :n] = f(z[:, :n] + bias) with the two-piece activation f of pointwise.cu, whose numbers (p, q) are the
        stored tensor `pq`; the further columns of out become 1, 0, 0, ... (a bias column for the product that reads it)."""
        if z.stride(1) != 1 or out.stride(1) != 1 or z.shape[1] < n or out.shape[1] < n or z.dtype != out.dtype \
                or bias.numel() != n or pq.numel() != 2 or bias.dtype != pq.dtype or z.shape[0] != out.shape[0]:
            raise KernelError("bias_xielu: z [rows, >= n], bias [n], pq [2] of one type, out [rows, >= n] of z's type")
        self.launches += 1
        self._check(self.lib.braid_bias_xielu(z.data_ptr(), z.stride(0), bias.data_ptr(), pq.data_ptr(), dtype_code(bias.dtype),
                                              out.data_ptr(), out.stride(0), dtype_code(out.dtype), z.shape[0], n, out.shape[1],
                                              self._stream()), "bias_xielu")

    @staticmethod
    def _check_head_extras(head_sinks, head_gate, nqh: int, dtype, head_scale=None) -> None:
        if head_scale is not None and (head_scale.dtype != torch.float32 or head_scale.numel() != nqh or not head_scale.is_contiguous()):
            raise KernelError(f"attention: a factor a head is a contiguous float32 tensor of {nqh} numbers")
        if head_sinks is not None and (head_sinks.dtype != torch.float32 or head_sinks.numel() != nqh or not head_sinks.is_contiguous()):
            raise KernelError(f"attention: a sink a head is a contiguous float32 tensor of {nqh} scores")
        if head_gate is not None and (head_gate.dtype != dtype or head_gate.stride(1) != 1 or head_gate.shape[1] < nqh):
            raise KernelError("attention: the heads' gates are rows of the result's element type with a column a head")

    @staticmethod
    def attn_mma_supports(head_dim: int) -> bool:
        return head_dim % 16 == 0 and 16 <= head_dim <= 256

    @staticmethod
    def attn_value_heads_a_launch(head_dim: int, value_heads: int) -> int:
        """How many kv heads' values a query head reads in one launch of the mma.sync kernel: as many as its
        float32 accumulators hold (value heads x head_dim up to 256), a divisor of `value_heads`."""
        return max(d for d in range(1, value_heads + 1) if value_heads % d == 0 and (d == 1 or d * head_dim <= 256))

    def attn_mma_library(self, head_dim: int, value_heads: int = 1):
        """The attention library for one head size (and, `value_heads` > 1, for a query head that reads the values
        of that many kv heads a launch), compiled at first use."""
        key = head_dim if value_heads == 1 else (head_dim, value_heads)
        lib = self._attn_libs.get(key)
        if lib is None:
            if not self.attn_mma_supports(head_dim):
                raise KernelError(f"the tensor-core attention takes head sizes in steps of 16 up to 256, not {head_dim}")
            lib = ctypes.CDLL(str(build.attention_library(head_dim, verbose=self._verbose, value_heads=value_heads)))
            lib.braid_last_error.restype = c_char_p
            lib.braid_attn_mma.restype = c_int
            lib.braid_attn_mma.argtypes = [c_void_p] * 9 + [c_int] * 13 + [c_float, c_int, c_float, c_float, c_void_p, c_void_p,
                                           c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
            lib.braid_attn_mma_partial_floats.restype = c_longlong
            lib.braid_attn_mma_partial_floats.argtypes = [c_int, c_int, c_int]
            if lib.braid_attn_mma_value_heads() != value_heads:
                raise KernelError("the attention library was built for another number of value heads")
            lib.has_tc = False
            if value_heads == 1:
                lib.braid_attn_tc_supported.restype = c_int
                lib.has_tc = bool(lib.braid_attn_tc_supported())
            if lib.has_tc:
                lib.braid_attn_tc.restype = c_int
                lib.braid_attn_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong] + [c_void_p] * 4 + [c_int] * 10 + \
                                             [c_float, c_int, c_float, c_float, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
            lib.braid_attn_mma_decode_slots.restype = c_int
            lib.braid_attn_mma_decode_slots.argtypes = [c_int]
            lib.decode_slots = lib.braid_attn_mma_decode_slots(1)     # CTAs of the few-token kernel held at once
            self._attn_libs[key] = lib
        return lib

    @staticmethod
    def _check_pages(cache: torch.Tensor) -> None:
        """The tensor-core attention kernels tile pages at compile time (csrc/page.h)."""
        if cache.dim() != 5 or cache.shape[3] != build.page_size():
            raise KernelError(f"the tensor-core attention reads a cache [pages, 2, kv_heads, {build.page_size()}, "
                              f"head_dim]; got {tuple(cache.shape)}")

    @staticmethod
    def attn_tc_supports(head_dim: int) -> bool:
        return head_dim in (64, 128)

    def attn_tc(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                q_start: torch.Tensor, q_len: torch.Tensor, kv_before: torch.Tensor, n_seqs: int, max_q_len: int,
                nqh: int, nkh: int, hd: int, window: Optional[int], scale: float, sink: Optional[float] = None,
                out_scale: float = 1.0, head_sinks: Optional[torch.Tensor] = None,
                head_gate: Optional[torch.Tensor] = None) -> None:
        """bfloat16 attention of prompts over the cache on tcgen05 (head sizes 64 and 128); `sink`, `head_sinks`,
        `out_scale` and `head_gate` as in `attn_simple`."""
        lib = self.attn_mma_library(hd)
        self._check_head_extras(head_sinks, head_gate, nqh, out.dtype)
        self._check_pages(cache)
        if not lib.has_tc:
            raise KernelError(f"the tcgen05 attention is built for head sizes 64 and 128, not {hd}")
        self.launches += 1
        cache_rows = cache.shape[0] * cache.shape[1] * cache.shape[2] * cache.shape[3]
        rc = lib.braid_attn_tc(q.data_ptr(), out.data_ptr(), cache.data_ptr(), cache_rows, page_table.data_ptr(),
                               q_start.data_ptr(), q_len.data_ptr(), kv_before.data_ptr(), q.stride(0), out.stride(0),
                               out.shape[0], n_seqs, max_q_len, nqh, nkh, hd, page_table.shape[1], int(window or 0),
                               float(scale), int(sink is not None), float(sink or 0.0), float(out_scale),
                               _ptr(head_sinks), _ptr(head_gate), head_gate.stride(0) if head_gate is not None else 0,
                               self._error_flag.data_ptr() + 12, self._stream())
        if rc != 0:
            raise KernelError(f"attn_tc: {lib.braid_last_error().decode(errors='replace')} (code {rc})")

    def attn_decode_slots(self, head_dim: int, value_heads: int = 1) -> int:
        vh = self.attn_value_heads_a_launch(head_dim, value_heads) if value_heads > 1 else 1
        return self.attn_mma_library(head_dim, vh).decode_slots

    def attn_mma(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                 q_start: torch.Tensor, q_len: torch.Tensor, kv_before: torch.Tensor, token_seq: torch.Tensor,
                 n_seqs: int, max_q_len: int, nqh: int, nkh: int, hd: int, window: Optional[int], scale: float,
                 n_splits: int = 1, few_tokens: bool = False, sink: Optional[float] = None,
                 out_scale: float = 1.0, head_sinks: Optional[torch.Tensor] = None,
                 head_gate: Optional[torch.Tensor] = None, keep_first: int = 0,
                 head_scale: Optional[torch.Tensor] = None, value_heads: int = 1) -> None:
        """bfloat16 attention over the cache on the tensor cores; `n_splits` > 1 slices the
        context (for steps of few tokens) and merges the slices in a second kernel.  `sink`, `head_sinks`,
        `out_scale`, `head_gate`, `keep_first`, `head_scale` and `value_heads` as in `attn_simple` (the sink is counted
        once, where the slices merge; where the accumulators do not hold the values of all kv heads, groups of them
        go to CTAs of their own)."""
        vh = self.attn_value_heads_a_launch(hd, value_heads) if value_heads > 1 else 1
        lib = self.attn_mma_library(hd, vh)
        self._check_head_extras(head_sinks, head_gate, nqh, out.dtype, head_scale)
        self._check_pages(cache)
        rows = out.shape[0]
        if value_heads > 1 and (value_heads != nkh or out.shape[1] < nqh * nkh * hd):
            raise KernelError("attn_mma: a head reads the values of its own kv head or of all, and the result holds them")
        partial = None
        if n_splits > 1:
            need = lib.braid_attn_mma_partial_floats(rows, nqh * value_heads, n_splits)
            if self._attn_partial is None or self._attn_partial.numel() < need:
                self._attn_partial = torch.empty(max(need, 1 << 22), dtype=torch.float32, device="cuda")
                self.workspace_generation += 1
            partial = self._attn_partial
            self.launches += 1
        for vh0 in (0,):                       # one launch: the groups of value heads are part of its grid
            self.launches += 1
            rc = lib.braid_attn_mma(q.data_ptr(), out.data_ptr(), _ptr(partial), cache.data_ptr(), page_table.data_ptr(),
                                    q_start.data_ptr(), q_len.data_ptr(), kv_before.data_ptr(), token_seq.data_ptr(),
                                    q.stride(0), out.stride(0), rows, n_seqs, max_q_len, nqh, nkh, hd,
                                    page_table.shape[1], cache.shape[0], int(window or 0), n_splits,
                                    1 if few_tokens else 0, float(scale), int(sink is not None), float(sink or 0.0),
                                    float(out_scale), _ptr(head_sinks), _ptr(head_gate),
                                    head_gate.stride(0) if head_gate is not None else 0, int(keep_first or 0),
                                    _ptr(head_scale), vh0, value_heads if value_heads > 1 else 0,
                                    self._error_flag.data_ptr() + 16, self._stream())
            if rc != 0:
                raise KernelError(f"attn_mma: {lib.braid_last_error().decode(errors='replace')} (code {rc})")

    # ------------------------------------------------------------------ element-wise kernels of other models
    def dyt(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None, in_scale: float = 1.0) -> None:
        """Dynamic Tanh: out = tanh(alpha * (x * in_scale)) * w + b, x the float32 residual stream (out may be x)."""
        rows, width = out.shape
        if x.dtype != torch.float32:
            raise KernelError("dyt reads the float32 residual stream")
        if not (w.dtype == b.dtype == alpha.dtype):
            raise KernelError("dyt: weight, bias and alpha must have one element type")
        self.launches += 1
        self._check(self.lib.braid_dyt(x.data_ptr(), w.data_ptr(), b.data_ptr(), alpha.data_ptr(), dtype_code(w.dtype),
                                       out.data_ptr(), dtype_code(out.dtype), _ptr(row_index), rows, width,
                                       float(in_scale), self._stream()), "dyt")

    def softcap(self, logits: torch.Tensor, cap: float) -> None:
        """logits <- cap * tanh(logits / cap), in place (float32, contiguous)."""
        if logits.dtype != torch.float32 or not logits.is_contiguous():
            raise KernelError("softcap works in place on contiguous float32 logits")
        self.launches += 1
        self._check(self.lib.braid_softcap(logits.data_ptr(), logits.numel(), float(cap), self._stream()), "softcap")

    def concat2(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = [a[r], b[r]]: two float32 streams side by side, in out's element type."""
        rows, width = a.shape
        if a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != a.shape or tuple(out.shape) != (rows, 2 * width):
            raise KernelError("concat2 wants two float32 tensors of one shape and an output twice as wide")
        self.launches += 1
        self._check(self.lib.braid_concat2(a.data_ptr(), b.data_ptr(), out.data_ptr(), dtype_code(out.dtype), rows, width,
                                           self._stream()), "concat2")

    # ------------------------------------------------------------------ libraries of single kinds of parts
    def part_library(self, name: str):
        """The kernel library of one kind of part ("latent", "moe"), compiled and opened at first use."""
        lib = self._part_libs.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(build.part_library(name, verbose=self._verbose)))
            lib.braid_last_error.restype = c_char_p
            if name == "latent":
                lib.braid_latent_prep.argtypes = [c_void_p, c_longlong, c_int] + [c_void_p] * 7 + [c_int] * 10 + \
                                                 [c_float, c_int, c_void_p, c_void_p]
                lib.braid_gemm_heads.argtypes = [c_void_p] * 4 + [c_int] * 5 + [c_longlong] * 5 + [c_float, c_void_p]
                lib.braid_gemm_heads_mma.argtypes = [c_void_p] * 4 + [c_int] * 4 + [c_longlong] * 5 + [c_float, c_void_p]
                lib.braid_gemm_heads_mma.restype = c_int
                lib.braid_attn_latent_simple.argtypes = [c_void_p, c_void_p, c_int] + [c_void_p] * 4 + \
                                                        [c_longlong, c_longlong] + [c_int] * 8 + [c_float, c_void_p, c_void_p]
                names = ("braid_latent_prep", "braid_gemm_heads", "braid_attn_latent_simple")
            elif name == "scan":
                lib.braid_causal_conv.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                                                  c_void_p, c_longlong, c_longlong] + [c_void_p] * 4 + [c_int] * 5 + [c_void_p]
                lib.braid_linear_scan.argtypes = [c_void_p, c_longlong] * 4 + [c_void_p] * 3 + [c_void_p, c_longlong] + \
                                                 [c_void_p, c_longlong, c_longlong] + [c_void_p] * 3 + [c_int] * 7 + \
                                                 [c_float, c_float, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int,
                                                  c_void_p]
                lib.braid_mlstm_gates.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_longlong,
                                                  c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]
                lib.braid_mlstm_out.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                                                c_longlong, c_void_p] + [c_int] * 4 + [c_float, c_void_p]
                lib.braid_scan_decay.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
                lib.braid_linear_scan_work_floats.argtypes = [c_int] * 7
                lib.braid_linear_scan_work_floats.restype = c_longlong
                lib.braid_gated_norm.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong,
                                                 c_void_p] + [c_int] * 5 + [c_float, c_float, c_void_p]
                names = ("braid_causal_conv", "braid_linear_scan", "braid_gated_norm", "braid_scan_decay", "braid_mlstm_gates",
                         "braid_mlstm_out")
            elif name == "moe":
                lib.braid_moe_route.argtypes = [c_void_p] * 3 + [c_int] * 5 + [c_float, c_int, c_void_p]
                lib.braid_moe_plan.argtypes = [c_void_p] * 6 + [c_int] * 5 + [c_void_p]
                lib.braid_moe_gemm_simt.argtypes = [c_void_p] * 7 + [c_int, c_int, c_longlong, c_longlong] + [c_int] * 5 + \
                                                   [c_void_p, c_void_p]
                lib.braid_moe_combine.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_longlong, c_void_p]
                lib.braid_moe_gemm_mma.argtypes = [c_void_p] * 7 + [c_int, c_longlong, c_longlong] + [c_int] * 5 + \
                                                  [c_void_p, c_void_p]
                lib.braid_moe_gemm_mma.restype = c_int
                names = ("braid_moe_route", "braid_moe_plan", "braid_moe_gemm_simt", "braid_moe_combine")
            else:
                names = ()
            for n in names:
                getattr(lib, n).restype = c_int
            self._part_libs[name] = lib
        return lib

    @staticmethod
    def _check_lib(lib, rc: int, what: str) -> None:
        if rc != 0:
            raise KernelError(f"{what}: {lib.braid_last_error().decode(errors='replace')} (code {rc})")

    # ------------------------------------------------------------------ latent attention
    def latent_prep(self, proj: torch.Tensor, q_cols: int, norm_w: torch.Tensor, inv_freq: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, page_table: Optional[torch.Tensor],
                    cache: Optional[torch.Tensor], q_lat: torch.Tensor, heads: int, dim: int, rot: int, rank: int,
                    rot_dims: int, page_size: int, eps: float, adjacent: bool = False) -> None:
        """A step's projected rows [rows, heads*(dim+rot) + rank + rot (+ more)]: the latent part is RMS-normed and,
        with the rotated shared key part, written into `cache` ([pages, 1, 1, page_size, rank + rot]); the rotated
        parts of the queries are written into q_lat[:, :, rank:] ([rows, heads, rank + rot])."""
        lib = self.part_library("latent")
        if cache is None:
            norm_w = None                       # no latent is made: the rows need not hold one
        elif norm_w is None:
            raise KernelError("latent_prep: the latent's norm weight is missing")
        if (norm_w is not None and norm_w.dtype != proj.dtype) or q_lat.dtype != proj.dtype or (cache is not None and cache.dtype != proj.dtype):
            raise KernelError("latent_prep: rows, norm weight, queries and cache must have one element type")
        if not q_lat.is_contiguous() or tuple(q_lat.shape) != (proj.shape[0], heads, rank + rot):
            raise KernelError(f"latent_prep: q_lat must be contiguous [{proj.shape[0]}, {heads}, {rank + rot}]")
        if cache is not None and (cache.dim() != 5 or cache.shape[1] != 1 or cache.shape[2] != 1 or cache.shape[3] != page_size
                                  or cache.shape[4] != rank + rot):
            raise KernelError(f"latent_prep: the cache must be [pages, 1, 1, {page_size}, {rank + rot}], got {tuple(cache.shape)}")
        cols = page_table.shape[1] if page_table is not None else 0
        self.launches += 1
        self._check_lib(lib, lib.braid_latent_prep(
            proj.data_ptr(), proj.stride(0), q_cols, _ptr(norm_w), inv_freq.data_ptr(), positions.data_ptr(),
            token_seq.data_ptr(), _ptr(page_table), _ptr(cache), q_lat.data_ptr(), dtype_code(proj.dtype),
            proj.shape[0], heads, dim, rot, rank, rot_dims, page_size, cols, cache.shape[0] if cache is not None else 0,
            float(eps), int(adjacent), self._error_flag.data_ptr(), self._stream()), "latent_prep")

    def gemm_heads(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                   mult: float = 1.0, tensor_cores: bool = True) -> None:
        """out[n, h, :] = w[h] x[n, h, :] for every head: x [rows, heads, K] and out [rows, heads, J] may be views
        (last dimension contiguous), w [heads, J, K] contiguous.  `gate` [rows, heads] (a view is fine): the result is
        multiplied by mult * sigmoid(gate).  bfloat16 operands whose rows start on 16 bytes run on the tensor cores
        unless `tensor_cores` is false; everything else on the plain kernel."""
        lib = self.part_library("latent")
        rows, heads, k = x.shape
        if w.dim() != 3 or w.shape[0] != heads or w.shape[2] != k or not w.is_contiguous():
            raise KernelError(f"gemm_heads: w must be contiguous [{heads}, J, {k}], got {tuple(w.shape)}")
        j = w.shape[1]
        if tuple(out.shape) != (rows, heads, j) or x.stride(2) != 1 or out.stride(2) != 1:
            raise KernelError("gemm_heads: shapes do not fit or last dimensions are not contiguous")
        if not (x.dtype == w.dtype == out.dtype) or (gate is not None and gate.dtype != x.dtype):
            raise KernelError("gemm_heads: every operand must have one element type")
        if gate is not None and (tuple(gate.shape) != (rows, heads) or gate.stride(1) != 1):
            raise KernelError("gemm_heads: gate must be [rows, heads] with contiguous heads")
        self.launches += 1
        if (tensor_cores and x.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0):
            self._check_lib(lib, lib.braid_gemm_heads_mma(
                x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(gate), rows, heads, j, k, x.stride(0), x.stride(1),
                out.stride(0), out.stride(1), gate.stride(0) if gate is not None else 0, float(mult), self._stream()),
                "gemm_heads_mma")
            return
        self._check_lib(lib, lib.braid_gemm_heads(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(gate), dtype_code(x.dtype), rows, heads, j, k,
            x.stride(0), x.stride(1), out.stride(0), out.stride(1), gate.stride(0) if gate is not None else 0,
            float(mult), self._stream()), "gemm_heads")

    def attn_latent_simple(self, q_lat: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                           positions: torch.Tensor, token_seq: torch.Tensor, rank: int, window: Optional[int],
                           scale: float) -> None:
        """Multi-query attention over the latent cache, one warp per (token, head): q_lat [rows, heads, D],
        out [rows, heads, rank], cache [pages, 1, 1, page_size, D]; a cached row is the key, its first `rank`
        numbers the value."""
        lib = self.part_library("latent")
        rows, heads, d = q_lat.shape
        if not q_lat.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (rows, heads, rank):
            raise KernelError("attn_latent_simple: q_lat [rows, heads, D] and out [rows, heads, rank] must be contiguous")
        if cache.dim() != 5 or cache.shape[1] != 1 or cache.shape[2] != 1 or cache.shape[4] != d or cache.dtype != q_lat.dtype:
            raise KernelError(f"attn_latent_simple: the cache must be [pages, 1, 1, page_size, {d}] of the queries' type")
        self.launches += 1
        self._check_lib(lib, lib.braid_attn_latent_simple(
            q_lat.data_ptr(), out.data_ptr(), dtype_code(out.dtype), cache.data_ptr(), page_table.data_ptr(),
            positions.data_ptr(), token_seq.data_ptr(), q_lat.stride(0), out.stride(0), rows, heads, d, rank,
            cache.shape[3], page_table.shape[1], cache.shape[0], int(window or 0), float(scale),
            self._error_flag.data_ptr() + 16, self._stream()), "attn_latent_simple")

    # ------------------------------------------------------------------ mixture of experts
    def moe_route(self, logits: torch.Tensor, idx: torch.Tensor, wgt: torch.Tensor, groups: int, keep: int,
                  mult: float = 1.0, sigmoid: bool = False) -> None:
        """Router logits [rows, experts] (float32) -> for each row its `top` experts idx [rows, top] (int32, by falling
        score) and their weights wgt [rows, top] (float32): softmax scores of the chosen, over their sum, times mult;
        with `sigmoid` the scores are sigmoids of the logits and the weights the chosen scores as they are, times mult."""
        lib = self.part_library("moe")
        rows, experts = logits.shape
        top = idx.shape[1]
        if logits.dtype != torch.float32 or not logits.is_contiguous() or idx.dtype != torch.int32 or wgt.dtype != torch.float32 \
                or tuple(idx.shape) != (rows, top) or tuple(wgt.shape) != (rows, top) or not idx.is_contiguous() or not wgt.is_contiguous():
            raise KernelError("moe_route: logits float32 [rows, experts], idx int32 and wgt float32 [rows, top], contiguous")
        self.launches += 1
        self._check_lib(lib, lib.braid_moe_route(logits.data_ptr(), idx.data_ptr(), wgt.data_ptr(), rows, experts, top,
                                                 groups, keep, float(mult), int(sigmoid), self._stream()), "moe_route")

    @staticmethod
    def moe_max_tiles(rows: int, top: int, experts: int, tile: int) -> int:
        """An upper bound of the tiles a step's plan uses: every tile holds a pair, and every expert wastes
        less than a tile."""
        pairs = rows * top
        return max(1, min(pairs, (pairs + min(experts, pairs) * (tile - 1)) // tile))

    def moe_plan(self, idx: torch.Tensor, token_seq: torch.Tensor, experts: int, tile: int):
        """Sort the (row, choice) pairs by expert, every expert's run padded to a multiple of `tile` slots.
        Returns (slot_pair [max_tiles*tile], pair_slot [rows*top], tile_expert [max_tiles], meta [1], max_tiles)."""
        lib = self.part_library("moe")
        rows, top = idx.shape
        max_tiles = self.moe_max_tiles(rows, top, experts, tile)
        buf = torch.empty(max_tiles * tile + rows * top + max_tiles + 4, dtype=torch.int32, device=idx.device)
        slot_pair = buf[:max_tiles * tile]
        pair_slot = buf[max_tiles * tile:max_tiles * tile + rows * top]
        tile_expert = buf[max_tiles * tile + rows * top:max_tiles * tile + rows * top + max_tiles]
        meta = buf[max_tiles * tile + rows * top + max_tiles:]
        self.launches += 1
        self._check_lib(lib, lib.braid_moe_plan(idx.data_ptr(), token_seq.data_ptr(), slot_pair.data_ptr(),
                                                pair_slot.data_ptr(), tile_expert.data_ptr(), meta.data_ptr(), rows, top,
                                                experts, tile, max_tiles, self._stream()), "moe_plan")
        return slot_pair, pair_slot, tile_expert, meta, max_tiles

    def moe_gemm_simt(self, x: torch.Tensor, w0: torch.Tensor, w1: Optional[torch.Tensor], out: torch.Tensor, plan,
                      top: int, tile: int, relu2: bool = False, in_wgt: Optional[torch.Tensor] = None) -> None:
        """`in_wgt` (float32 [rows, top], with w1): a pair's weight multiplies the expert's input, that is gate and up
        before the activation.  The experts' products over a plan's slots, plain.  With w1: out[slot] = silu(w0[e] x[row]) * (w1[e] x[row]),
        x the step's rows; without: out[slot] = w0[e] x[slot], x a tensor of slots; with `relu2` (and no w1):
        out[slot] = relu(w0[e] x[row])^2, x the step's rows (experts without a gate).  w0, w1 [experts, J, K]."""
        lib = self.part_library("moe")
        slot_pair, _pair_slot, tile_expert, meta, max_tiles = plan
        j, k = w0.shape[1], w0.shape[2]
        if not w0.is_contiguous() or (w1 is not None and (not w1.is_contiguous() or w1.shape != w0.shape)):
            raise KernelError("moe_gemm: expert weights must be contiguous [experts, J, K]")
        if x.shape[1] != k or out.shape[1] != j or out.shape[0] != max_tiles * tile or x.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("moe_gemm: shapes do not fit")
        if not (x.dtype == w0.dtype == out.dtype):
            raise KernelError("moe_gemm: every operand must have one element type")
        self.launches += 1
        self._check_lib(lib, lib.braid_moe_gemm_simt(
            x.data_ptr(), w0.data_ptr(), _ptr(w1), out.data_ptr(), slot_pair.data_ptr(), tile_expert.data_ptr(),
            meta.data_ptr(), dtype_code(x.dtype), self._moe_mode(w1, relu2), x.stride(0), out.stride(0), j, k, top, tile,
            max_tiles, self._in_wgt(in_wgt, x, top, w1), self._stream()), "moe_gemm_simt")

    @staticmethod
    def _in_wgt(in_wgt, x, top: int, w1):
        if in_wgt is None:
            return None
        if w1 is None or in_wgt.dtype != torch.float32 or not in_wgt.is_contiguous() or tuple(in_wgt.shape) != (x.shape[0], top):
            raise KernelError("moe_gemm: the weights on the experts' input are float32 [rows, top] and go with the gated product")
        return in_wgt.data_ptr()

    @staticmethod
    def _moe_mode(w1, relu2: bool) -> int:
        if relu2 and w1 is not None:
            raise KernelError("moe_gemm: the squared relu is the activation of experts without a gate (no w1)")
        return 2 if relu2 else (0 if w1 is not None else 1)

    @staticmethod
    def moe_gemm_mma_eligible(x: torch.Tensor, w0: torch.Tensor, tile: int) -> bool:
        return (x.dtype == torch.bfloat16 and w0.dtype == torch.bfloat16 and w0.shape[2] % 8 == 0 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w0.data_ptr() % 16 == 0 and tile in (16, 64))

    def moe_gemm_mma(self, x: torch.Tensor, w0: torch.Tensor, w1: Optional[torch.Tensor], out: torch.Tensor, plan,
                     top: int, tile: int, relu2: bool = False, in_wgt: Optional[torch.Tensor] = None) -> None:
        """`moe_gemm_simt` in bfloat16 on the tensor cores; the plan's tile (16 or 64 slots) is the CTA's."""
        lib = self.part_library("moe")
        slot_pair, _pair_slot, tile_expert, meta, max_tiles = plan
        j, k = w0.shape[1], w0.shape[2]
        if not self.moe_gemm_mma_eligible(x, w0, tile) or not w0.is_contiguous() or (w1 is not None and (
                not w1.is_contiguous() or w1.shape != w0.shape or w1.dtype != w0.dtype or w1.data_ptr() % 16)):
            raise KernelError("moe_gemm_mma: bfloat16 operands, k and row strides in multiples of 8, starts on 16 bytes")
        if x.shape[1] != k or out.shape[1] != j or out.shape[0] != max_tiles * tile or out.dtype != torch.bfloat16 \
                or x.stride(1) != 1 or out.stride(1) != 1 or out.data_ptr() % 4:
            raise KernelError("moe_gemm_mma: shapes do not fit")
        self.launches += 1
        self._check_lib(lib, lib.braid_moe_gemm_mma(
            x.data_ptr(), w0.data_ptr(), _ptr(w1), out.data_ptr(), slot_pair.data_ptr(), tile_expert.data_ptr(),
            meta.data_ptr(), self._moe_mode(w1, relu2), x.stride(0), out.stride(0), j, k, top, tile, max_tiles,
            self._in_wgt(in_wgt, x, top, w1), self._stream()), "moe_gemm_mma")

    @staticmethod
    def attn_latent_mma_supports(rank: int, rot: int) -> bool:
        """Latent sizes the tensor-core attention is compiled for: kv_rank and rot_dim in multiples of 16, a rank
        above 256 in multiples of 256, and a query tile plus two key tiles within one SM's shared memory."""
        return (rank % 16 == 0 and rot % 16 == 0 and rank > 0 and (rank <= 256 or rank % 256 == 0)
                and 128 * (rank + rot + 8) * 2 <= 227 * 1024)

    def latent_attention_library(self, rank: int, rot: int):
        key = ("latattn", rank, rot)
        lib = self._part_libs.get(key)
        if lib is None:
            if not self.attn_latent_mma_supports(rank, rot):
                raise KernelError(f"the tensor-core latent attention is not built for kv_rank {rank}, rot_dim {rot}")
            lib = ctypes.CDLL(str(build.latent_attention_library(rank, rot, verbose=self._verbose)))
            lib.braid_last_error.restype = c_char_p
            lib.braid_latent_attn_mma.restype = c_int
            lib.braid_latent_attn_mma.argtypes = [c_void_p] * 9 + [c_int] * 8 + [c_float, c_void_p, c_void_p]
            lib.braid_latent_attn_partial_floats.restype = c_longlong
            lib.braid_latent_attn_partial_floats.argtypes = [c_int, c_int, c_int]
            lib.vparts = lib.braid_latent_attn_vparts()
            lib.braid_latent_attn_tile_rows.restype = c_int
            lib.braid_latent_attn_tile_rows.argtypes = [c_int, c_int]
            if (lib.braid_latent_attn_rank(), lib.braid_latent_attn_rot()) != (rank, rot):
                raise KernelError("the latent attention library was built for another size")
            self._part_libs[key] = lib
        return lib

    def attn_latent_ctas(self, rank: int, rot: int, n_seqs: int, max_q_len: int, heads: int) -> int:
        """CTAs of the tensor-core latent attention for a step, before the context is sliced: steps of few
        (token, head) pairs run tiles of 16 rows whose warps share the rows, others tiles of 64 (and, for a
        rank above 256, one CTA a part of 256 value columns)."""
        lib = self.latent_attention_library(rank, rot)
        tile = lib.braid_latent_attn_tile_rows(max_q_len, heads)
        return n_seqs * -(-max_q_len * heads // tile) * (1 if tile == 16 else lib.vparts)

    def attn_latent_mma(self, q_lat: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                        q_start: torch.Tensor, q_len: torch.Tensor, kv_before: torch.Tensor, token_seq: torch.Tensor,
                        n_seqs: int, max_q_len: int, rank: int, window: Optional[int], scale: float,
                        n_splits: int = 1) -> None:
        """`attn_latent_simple` in bfloat16 on the tensor cores.  Rows of padding are not written.  `n_splits` > 1
        slices the context (steps of few tokens) and merges the slices in a second kernel."""
        rows, heads, d = q_lat.shape
        lib = self.latent_attention_library(rank, d - rank)
        self._check_pages(cache)
        if q_lat.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
                or not q_lat.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (rows, heads, rank) \
                or cache.dim() != 5 or cache.shape[1] != 1 or cache.shape[2] != 1 or cache.shape[4] != d:
            raise KernelError("attn_latent_mma: contiguous bfloat16 q_lat [rows, heads, D], out [rows, heads, rank] and "
                              "a cache [pages, 1, 1, page_size, D]")
        partial = None
        if n_splits > 1:
            need = lib.braid_latent_attn_partial_floats(rows, heads, n_splits)
            if self._attn_partial is None or self._attn_partial.numel() < need:
                self._attn_partial = torch.empty(max(need, 1 << 22), dtype=torch.float32, device="cuda")
                self.workspace_generation += 1
            partial = self._attn_partial
            self.launches += 1
        self.launches += 1
        self._check_lib(lib, lib.braid_latent_attn_mma(
            q_lat.data_ptr(), out.data_ptr(), _ptr(partial), cache.data_ptr(), page_table.data_ptr(), q_start.data_ptr(),
            q_len.data_ptr(), kv_before.data_ptr(), token_seq.data_ptr(), rows, n_seqs, max_q_len, heads,
            page_table.shape[1], cache.shape[0], int(window or 0), n_splits, float(scale),
            self._error_flag.data_ptr() + 16, self._stream()), "attn_latent_mma")

    def moe_combine(self, h: torch.Tensor, y: torch.Tensor, plan, wgt: Optional[torch.Tensor], top: Optional[int] = None) -> None:
        """h[row] += sum_k wgt[row, k] * y[slot of (row, k)], float32, choices added in their order (wgt None: every
        weight is 1, and `top` says how many choices a row has)."""
        lib = self.part_library("moe")
        rows, width = h.shape
        if h.dtype != torch.float32 or not h.is_contiguous() or y.shape[1] != width or y.stride(1) != 1:
            raise KernelError("moe_combine: h is the contiguous float32 residual stream, y [slots, width]")
        self.launches += 1
        self._check_lib(lib, lib.braid_moe_combine(h.data_ptr(), y.data_ptr(), dtype_code(y.dtype), plan[1].data_ptr(),
                                                   _ptr(wgt), rows, width, wgt.shape[1] if wgt is not None else int(top),
                                                   y.stride(0), self._stream()),
                        "moe_combine")

    # ------------------------------------------------------------------ mixers with a recurrent state
    @staticmethod
    def _state_args(state: torch.Tensor, offset: int):
        if state.dtype != torch.uint8 or state.dim() != 2 or state.stride(1) != 1:
            raise KernelError("a state area is a uint8 tensor [slots, bytes]")
        return state.data_ptr(), state.stride(0), int(offset)

    def causal_conv(self, x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], state: torch.Tensor,
                    state_offset: int, ctx, silu: bool = True) -> None:
        """y[t, c] = act(b[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]) along each sequence of the step (x, y
        [rows, channels], views are fine; w [channels, taps]); inputs before the step come from the state
        (float32 [taps - 1, channels] at `state_offset` bytes of each slot), which is then moved on."""
        lib = self.part_library("scan")
        rows, channels = y.shape
        taps = w.shape[1]
        if not (x.dtype == y.dtype == w.dtype) or (b is not None and b.dtype != x.dtype) or x.stride(1) != 1 \
                or y.stride(1) != 1 or not w.is_contiguous() or w.shape[0] != channels or x.shape[1] != channels:
            raise KernelError("causal_conv: x, y, w, b of one element type; w contiguous [channels, taps]")
        self.launches += 2 if taps > 1 else 1
        self._check_lib(lib, lib.braid_causal_conv(
            x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), w.data_ptr(), _ptr(b), dtype_code(x.dtype),
            *self._state_args(state, state_offset), ctx.token_seq.data_ptr(), ctx.q_start.data_ptr(),
            ctx.q_len.data_ptr(), ctx.slot_ids.data_ptr(), rows, ctx.n_seqs, channels, taps, int(silu), self._stream()),
            "causal_conv")

    def linear_scan(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, gate_bias: torch.Tensor,
                    out: torch.Tensor, state: torch.Tensor, state_offset: int, ctx, heads: int, groups: int, dk: int,
                    dv: int, mode: str, q_scale: float = 1.0, inv_tau: float = 1.0, a_log: Optional[torch.Tensor] = None,
                    skip: Optional[torch.Tensor] = None, chunk: Optional[int] = None, gate_is_decay: bool = False,
                    kappa: Optional[torch.Tensor] = None, v_cols: Optional[int] = None) -> None:
        """The recurrence S <- diag(a) S + (kappa k) v^T, o = S^T (q_scale q) + skip v, token by token along each
        sequence of the step, S float32 [heads, dk, dv] at `state_offset` bytes of each slot.  mode "channel":
        a = sigmoid(gate + gate_bias)^inv_tau per key channel (gate float32 [rows, heads * dk]); mode "head":
        dt = softplus(gate + gate_bias), a = exp(-exp(a_log) dt), kappa = dt (gate [rows, heads] in the run's
        type).  q, k [rows, groups * dk], v [rows, heads * dv] (views are fine); out float32 [rows, heads * dv].
        `gate_is_decay` (mode "channel"): `gate` holds the decays themselves, as `scan_decay` left them.
        mode "given": a = gate[row, head] and kappa = kappa[row, head], float32 views of one row stride, worked out
        before (`mlstm_gates`); with `v_cols` < dv, v holds v_cols columns a head and the state's other columns take
        a value of 1 (a normaliser: S[:, v_cols] sums the decayed keys, out[:, v_cols] is its product with the query).
        `gate_bias` is then unused (pass any tensor of the rows' type).
        A step whose longest sequence brings at least two chunks of `chunk` tokens (default: see SCAN_CHUNK; 0: never)
        walks its chunks side by side in three passes (see csrc/scan.cu); the results differ from the walk
        token by token by rounding only."""
        lib = self.part_library("scan")
        if not (q.dtype == k.dtype == v.dtype == gate_bias.dtype) or out.dtype != torch.float32 \
                or any(t.stride(1) != 1 for t in (q, k, v, gate, out)):
            raise KernelError("linear_scan: q, k, v and the gate's bias of one element type, out float32, rows contiguous")
        if mode == "channel":
            if gate.dtype != torch.float32 or gate.shape[1] != heads * dk or gate_bias.numel() != heads * dk:
                raise KernelError("linear_scan: a decay per channel takes a float32 gate [rows, heads * dk]")
        elif mode == "head":
            if gate.dtype != q.dtype or gate.shape[1] != heads or gate_bias.numel() != heads or a_log is None \
                    or a_log.dtype != q.dtype or (skip is not None and skip.dtype != q.dtype):
                raise KernelError("linear_scan: a decay per head takes a gate [rows, heads], its bias, A_log and a skip "
                                  "of the rows' element type")
        elif mode == "given":
            if gate.dtype != torch.float32 or kappa is None or kappa.dtype != torch.float32 or kappa.stride(0) != gate.stride(0) \
                    or kappa.stride(1) != 1 or gate.shape[1] < heads or kappa.shape[1] < heads:
                raise KernelError("linear_scan: given decays and key factors are float32 [rows, heads] views of one row stride")
        else:
            raise KernelError(f"linear_scan: unknown decay mode {mode!r}")
        vc = dv if v_cols is None else int(v_cols)
        if v.shape[1] < heads * vc or out.shape[1] < heads * dv:
            raise KernelError("linear_scan: v or out does not hold the heads' columns")
        if chunk is None:
            chunk = SCAN_CHUNK if SCAN_CHUNK is not None else (128 if int(ctx.max_q_len) >= 1024 else 64)
        chunk = int(chunk)
        code = {"channel": 0, "head": 1, "given": 2}[mode]
        need = lib.braid_linear_scan_work_floats(ctx.n_seqs, int(ctx.max_q_len), chunk, heads, dk, dv, code)
        work = torch.empty(need, dtype=torch.float32, device=out.device) if need > 0 else None
        self.launches += 3 if need > 0 else 1
        self._check_lib(lib, lib.braid_linear_scan(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), gate.data_ptr(), gate.stride(0),
            gate_bias.data_ptr(), _ptr(a_log), _ptr(skip), out.data_ptr(), out.stride(0),
            *self._state_args(state, state_offset), ctx.q_start.data_ptr(), ctx.q_len.data_ptr(), ctx.slot_ids.data_ptr(),
            dtype_code(q.dtype), code, ctx.n_seqs, heads, groups, dk, dv, float(q_scale),
            float(inv_tau), int(ctx.max_q_len), chunk, _ptr(work), need, int(gate_is_decay), _ptr(kappa), vc,
            self._stream()), "linear_scan")

    def mlstm_gates(self, z: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, out: torch.Tensor,
                    state: torch.Tensor, state_offset: int, ctx, heads: int, cap: float) -> None:
        """The gates of a matrix memory along each sequence of the step.  z float32 [rows, 2 heads]: the logits of the
        input gates, then of the forget gates (biases [heads] each).  li = cap tanh((zi + bi) / cap),
        lf = log sigmoid(cap tanh((zf + bf) / cap)); m_t = max(lf + m_(t-1), li) with m float32 [heads] at
        `state_offset` bytes of each slot (0 for a new sequence).  out float32 [rows, 3 heads]: exp(lf + m_(t-1) - m_t),
        exp(li - m_t), exp(-m_t)."""
        lib = self.part_library("scan")
        if z.dtype != torch.float32 or z.stride(1) != 1 or z.shape[1] < 2 * heads or out.dtype != torch.float32 \
                or not out.is_contiguous() or tuple(out.shape) != (z.shape[0], 3 * heads) or bias_i.dtype != bias_f.dtype \
                or bias_i.numel() != heads or bias_f.numel() != heads:
            raise KernelError("mlstm_gates: z float32 [rows, 2 heads], out contiguous float32 [rows, 3 heads], a bias a head")
        self.launches += 1
        self._check_lib(lib, lib.braid_mlstm_gates(
            z.data_ptr(), z.stride(0), bias_i.data_ptr(), bias_f.data_ptr(), dtype_code(bias_i.dtype), out.data_ptr(),
            *self._state_args(state, state_offset), ctx.q_start.data_ptr(), ctx.q_len.data_ptr(), ctx.slot_ids.data_ptr(),
            ctx.n_seqs, heads, float(cap), self._stream()), "mlstm_gates")

    def mlstm_out(self, y: torch.Tensor, floors: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                  token_seq: torch.Tensor, heads: int, dv: int, eps: float) -> None:
        """The read-out of a matrix memory: y float32 [rows, heads * (dv + 1)] (a head's S^T q, then n . q);
        o = y[:dv] / (max(|n . q|, floors[row, head]) + 1e-6); out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate),
        w [heads * dv], gate and out [rows, heads * dv] in the run's type (views are fine)."""
        lib = self.part_library("scan")
        rows = y.shape[0]
        if y.dtype != torch.float32 or not y.is_contiguous() or y.shape[1] != heads * (dv + 1) or floors.dtype != torch.float32 \
                or floors.stride(1) != 1 or not (gate.dtype == w.dtype == out.dtype) or gate.stride(1) != 1 or out.stride(1) != 1 \
                or w.numel() != heads * dv or gate.shape[1] < heads * dv or out.shape[1] < heads * dv:
            raise KernelError("mlstm_out: y contiguous float32 [rows, heads * (dv + 1)]; gate, w, out of one element type")
        self.launches += 1
        self._check_lib(lib, lib.braid_mlstm_out(
            y.data_ptr(), floors.data_ptr(), floors.stride(0), gate.data_ptr(), gate.stride(0), w.data_ptr(), out.data_ptr(),
            out.stride(0), token_seq.data_ptr(), dtype_code(out.dtype), rows, heads, dv, float(eps), self._stream()), "mlstm_out")

    def scan_decay(self, z: torch.Tensor, bias: torch.Tensor, inv_tau: float) -> None:
        """z <- sigmoid(z + bias)^inv_tau in place (z float32 [rows, n]): the decays of a recurrence from their logits,
        once for a long step instead of in every CTA of the recurrence."""
        lib = self.part_library("scan")
        if z.dtype != torch.float32 or z.stride(1) != 1 or bias.numel() != z.shape[1]:
            raise KernelError("scan_decay: z float32 [rows, n] with contiguous rows, bias of n numbers")
        self.launches += 1
        self._check_lib(lib, lib.braid_scan_decay(z.data_ptr(), z.stride(0), bias.data_ptr(), dtype_code(bias.dtype), z.shape[0],
                                                  z.shape[1], float(inv_tau), self._stream()), "scan_decay")

    def gated_norm(self, y: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, out: torch.Tensor, token_seq: torch.Tensor,
                   group: int, gate_first: bool, eps: float, out_scale: float = 1.0) -> None:
        """Groups of `group` columns of y (float32 [rows, width]), each by its own root mean square: norm then
        silu(gate), or (gate_first) silu(gate) then norm; times w (one weight a group's column, or one a column of
        the row) and out_scale."""
        lib = self.part_library("scan")
        rows, width = y.shape
        if y.dtype != torch.float32 or not y.is_contiguous() or not (gate.dtype == w.dtype == out.dtype) \
                or gate.stride(1) != 1 or out.stride(1) != 1 or w.numel() not in (group, width) or tuple(out.shape) != (rows, width):
            raise KernelError("gated_norm: y contiguous float32; gate, w, out of one element type; w of a group's or a row's length")
        self.launches += 1
        self._check_lib(lib, lib.braid_gated_norm(
            y.data_ptr(), gate.data_ptr(), gate.stride(0), w.data_ptr(), w.numel(), out.data_ptr(), out.stride(0),
            token_seq.data_ptr(), dtype_code(out.dtype), rows, width, group, int(gate_first), float(eps), float(out_scale),
            self._stream()), "gated_norm")

    # ------------------------------------------------------------------ matrix products
    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None) -> None:
        n, k = x.shape
        m = w.shape[0]
        if x.dtype != w.dtype:
            # the kernel reads both operands as one element type: a mixed call would read the
            # narrower operand past its end
            raise KernelError(f"gemm_simt: x is {x.dtype} and w is {w.dtype}; both operands must have one element type")
        if w.shape[1] != k or tuple(out.shape) != (n, m):
            raise KernelError(f"gemm_simt: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        mode = 1 if residual is not None else 0
        self.launches += 1
        self._check(self.lib.braid_gemm_simt(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual),
                                             dtype_code(x.dtype), dtype_code(out.dtype), mode, n, m, k,
                                             x.stride(0), w.stride(0), out.stride(0), self._stream()), "gemm_simt")

    def tc_workspace(self, nbytes: int) -> torch.Tensor:
        if self._tc_workspace is None or self._tc_workspace.numel() * 4 < nbytes:
            self._tc_workspace = torch.empty(max((nbytes + 3) // 4, 1 << 22), dtype=torch.float32, device="cuda")
            self.workspace_generation += 1
        return self._tc_workspace

    def _stream_k_workspace(self, n: int, w_rows: int, k: int, block_n: int) -> torch.Tensor:
        need = self.lib.braid_gemm_tc_workspace_bytes(n, w_rows, k, block_n)
        if need < 0:
            raise KernelError(f"gemm_tc: no stream-k plan for {n} rows x {w_rows} x {k} with token tile {block_n}")
        return self.tc_workspace(need)

    def gemm_tc(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                swiglu: bool = False, block_n: int = 0, stream_k: bool = False,
                in_scale: Optional[RowScale] = None, activation: str = "silu") -> None:
        """bfloat16 x [n, k] times w [m, k]^T on the tensor cores.  With `swiglu`, w holds
        gate and up rows interleaved in blocks of 16 (`interleave_gate_up`) and out is [n, I].  `stream_k` spreads the weight stream
        evenly over all SMs whatever the shape (for up to a few hundred tokens) and adds a reduce kernel.
        Whole tiles of more than 128 tokens run on pairs of SMs (`gemm_tc_pair`: faster at every
        measured size, and bit for bit the same result) unless `block_n` names a token tile.
        `in_scale`: a row scale that x still wants; the store and SwiGLU epilogues apply it to their results."""
        n, k = x.shape
        if not stream_k and block_n == 0 and token_tile(n) == PAIR_TOKEN_TILE and in_scale is None:
            return self.gemm_tc_pair(x, w, out, residual=residual, swiglu=swiglu, activation=activation)
        w_rows = w.shape[0]
        m = out.shape[1] if swiglu else w_rows
        if swiglu and w_rows != 2 * (-(-m // 16) * 16):
            raise KernelError(f"the SwiGLU epilogue wants {2 * (-(-m // 16) * 16)} interleaved weight rows for "
                              f"{m} outputs, got {w_rows} (see interleave_gate_up)")
        mode = (2 | activation_code(activation) << 4) if swiglu else (1 if residual is not None else 0)
        block_n = block_n or token_tile(n)
        ws = None
        if stream_k:
            if self.pending_partial is not None:
                raise KernelError("a deferred sum still lives in the GEMM workspace; resolve it before the next "
                                  "stream-k product")
            ws = self._stream_k_workspace(n, w_rows, k, block_n)
            self.launches += 1
        self.launches += 1
        self._check(self.lib.braid_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual), _ptr(ws),
                                           ws.numel() * 4 if ws is not None else 0,
                                           dtype_code(out.dtype), mode, n, m, k, x.stride(0), w.stride(0),
                                           out.stride(0), block_n, int(stream_k), None, *_scale_args(in_scale),
                                           _ptr(self._rs_rows(n, x.device) if stream_k and in_scale is not None else None),
                                           self._error_flag.data_ptr() + 4, self._stream()), "gemm_tc")

    @staticmethod
    def _rs_rows(n: int, device) -> torch.Tensor:
        """Room for every row's scale (a stream-k product with a row scale writes them for the adding-up)."""
        return torch.empty(-(-n // 4) * 4, dtype=torch.float32, device=device)

    def gemm_tc_pair(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                     residual: Optional[torch.Tensor] = None, swiglu: bool = False, direct_out: bool = False,
                     activation: str = "silu") -> None:
        """As `gemm_tc` with whole tiles, on pairs of SMs: tiles of 256 weight rows x 256 tokens, each CTA of
        a pair loading half of both operands (tcgen05.mma.cta_group::2).  For prompts.  The output leaves
        through TMA stores (a TMA reduce-add for a residual summed in place) where it can be addressed so;
        `direct_out` makes every thread store its own elements instead, as it does anyway otherwise."""
        n, k = x.shape
        w_rows = w.shape[0]
        m = out.shape[1] if swiglu else w_rows
        if swiglu and w_rows != 2 * (-(-m // 16) * 16):
            raise KernelError(f"the SwiGLU epilogue wants {2 * (-(-m // 16) * 16)} interleaved weight rows for "
                              f"{m} outputs, got {w_rows} (see interleave_gate_up)")
        mode = (2 | activation_code(activation) << 4) if swiglu else (1 if residual is not None else 0)
        self.launches += 1
        self._check(self.lib.braid_gemm_tc2(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual),
                                            dtype_code(out.dtype), mode, n, m, k, x.stride(0), w.stride(0),
                                            out.stride(0), int(direct_out), self._error_flag.data_ptr() + 4,
                                            self._stream()),
                    "gemm_tc_pair")

    def gemm_tc_partial(self, x: torch.Tensor, w: torch.Tensor, in_scale: Optional[RowScale] = None) -> "PartialProduct":
        """The stream-k product without its reduce: the partial products stay in the
        workspace, and the returned handle lets one of the `streamk_reduce*` calls add
        them up together with what follows.  Only one such handle may be open at a time."""
        if self.pending_partial is not None:
            raise KernelError("a deferred sum still lives in the GEMM workspace; resolve it first")
        n, k = x.shape
        w_rows = w.shape[0]
        block_n = token_tile(n)
        ws = self._stream_k_workspace(n, w_rows, k, block_n)
        plan = (c_int * 8)()
        rs = self._rs_rows(n, x.device) if in_scale is not None else None
        self.launches += 1
        self._check(self.lib.braid_gemm_tc(x.data_ptr(), w.data_ptr(), None, None, ws.data_ptr(), ws.numel() * 4,
                                           F32, 0, n, w_rows, k, x.stride(0), w.stride(0), 0, block_n, 1, plan,
                                           *_scale_args(in_scale), _ptr(rs),
                                           self._error_flag.data_ptr() + 4, self._stream()), "gemm_tc_partial")
        p = PartialProduct(ws, plan, n, w_rows, rs)
        self.pending_partial = p
        return p

    def _close_partial(self, p: "PartialProduct") -> None:
        if self.pending_partial is not p:
            raise KernelError("this partial product is not the one that lives in the workspace")
        self.pending_partial = None

    def streamk_reduce(self, p: "PartialProduct", out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                       swiglu: bool = False, activation: str = "silu") -> None:
        m = out.shape[1] if swiglu else p.w_rows
        mode = (2 | activation_code(activation) << 4) if swiglu else (1 if residual is not None else 0)
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce(p.workspace.data_ptr(), p.plan, p.n_rows, out.data_ptr(), _ptr(residual),
                                                  m, out.stride(0), dtype_code(out.dtype), mode, _ptr(p.rs_rows),
                                                  self._stream()),
                    "streamk_reduce")

    def streamk_reduce_norm(self, p: "PartialProduct", h: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float,
                            row_index: Optional[torch.Tensor] = None) -> None:
        """h += sum of the partial products (written back unless rows are gathered), then
        out = RMSNorm(h) * w, in one kernel."""
        rows_out, width = out.shape
        if p.rs_rows is not None:
            raise KernelError("this partial product carries a row scale, which reduce + norm does not apply")
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_norm(p.workspace.data_ptr(), p.plan, p.n_rows, h.data_ptr(), w.data_ptr(),
                                                       dtype_code(w.dtype), out.data_ptr(), dtype_code(out.dtype),
                                                       _ptr(row_index), rows_out, width, float(eps), self._stream()),
                    "streamk_reduce_norm")

    def streamk_reduce_rope_kv(self, p: "PartialProduct", qkv: torch.Tensor, inv_freq: torch.Tensor,
                               positions: torch.Tensor, token_seq: torch.Tensor, page_table: Optional[torch.Tensor],
                               cache: Optional[torch.Tensor], nqh: int, nkh: int, hd: int, rope_dim: int,
                               adjacent: bool, page_size: int) -> None:
        """qkv = sum of the partial products, rotated, keys and values into the cache."""
        cols = page_table.shape[1] if page_table is not None else 0
        num_pages = cache.shape[0] if cache is not None else 0
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_rope_kv(
            p.workspace.data_ptr(), p.plan, qkv.data_ptr(), inv_freq.data_ptr(), positions.data_ptr(),
            token_seq.data_ptr(), _ptr(page_table), _ptr(cache), qkv.shape[0], nqh, nkh, hd, rope_dim, int(adjacent),
            page_size, cols, num_pages, _ptr(p.rs_rows), self._error_flag.data_ptr(), self._stream()),
            "streamk_reduce_rope_kv")

    def streamk_reduce_prep(self, p: Optional["PartialProduct"], h: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                            eps: float) -> RowScale:
        """h += sum of the partial products (p None: h is complete), out = bfloat16(h * w), and the returned
        RowScale completes the RMSNorm of h with weights w: whoever multiplies `out` by a matrix applies it
        to its results (`in_scale`).  Many small CTAs instead of one per row."""
        rows, width = h.shape
        if out.dtype != torch.bfloat16 or h.dtype != torch.float32 or out.shape != h.shape:
            raise KernelError("reduce_prep reads the float32 residual stream and writes bfloat16 of the same shape")
        cols = self.lib.braid_streamk_reduce_prep_cols()
        shares = torch.empty((-(-width // cols), -(-rows // 4) * 4), dtype=torch.float32, device=h.device)
        if p is not None:
            if p.rs_rows is not None:
                raise KernelError("this partial product carries a row scale, which the residual sum does not apply")
            self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_prep(
            p.workspace.data_ptr() if p is not None else None, p.plan if p is not None else None, rows, h.data_ptr(),
            w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), shares.data_ptr(), shares.stride(0), width,
            self._stream()), "streamk_reduce_prep")
        return RowScale(shares, width, eps)

    @staticmethod
    def gemm_tc_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    # ------------------------------------------------------------------ token choice
    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        rows, vocab = logits.shape
        self.launches += 1
        self._check(self.lib.braid_argmax(logits.data_ptr(), logits.stride(0), out.data_ptr(), rows, vocab,
                                          self._error_flag.data_ptr() + 8, self._stream()), "argmax")

    def sample(self, logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor,
               uniform: torch.Tensor, top_k=None, top_p=None, min_p=None, rep_penalty=None,
               hist_off=None, hist_tok=None, hist_cnt=None, bias_off=None, bias_tok=None, bias_val=None) -> None:
        rows, vocab = logits.shape
        self.launches += 1
        self._check(self.lib.braid_sample(
            logits.data_ptr(), work.data_ptr(), logits.stride(0), out.data_ptr(), rows, vocab,
            temperature.data_ptr(), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(rep_penalty), uniform.data_ptr(),
            _ptr(hist_off), _ptr(hist_tok), _ptr(hist_cnt), _ptr(bias_off), _ptr(bias_tok), _ptr(bias_val),
            self._error_flag.data_ptr() + 8, self._stream()), "sample")


_KERNELS: Optional[Kernels] = None


def get_kernels(verbose: bool = True) -> Kernels:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = Kernels(verbose=verbose)
    return _KERNELS
