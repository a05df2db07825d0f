"""ctypes bindings of the kernel libraries: torch tensors in, launches on torch's current stream.

`KernelSet(dtype)` gives the launchers of one element type (float32: the true 32-bit set;
bfloat16: the serving set). Every wrapper checks device, dtype and contiguity before it passes a
pointer on, and raises on a non-zero return code. There is no CPU path: a tensor that is not on a
CUDA device is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library



class KernelError(RuntimeError):
    pass


def _ptr(t: torch.Tensor | None, dtype=None, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return c_void_p(t.data_ptr())


try:        # the raw handle of torch's current stream without building a Stream object (a launch costs microseconds)
    _raw_stream, _current_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:      # a torch without these entry points: the public, slower way
    _raw_stream = _current_device = None


def _stream():
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = [0]   # kernels enqueued through these bindings since import (a bench reads the difference)


def _check(code: int, what: str):
    LAUNCHES[0] += 1
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: arguments refused by the launcher (code {code})")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        rt = ctypes.CDLL("libcudart.so")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return "see cudaError_t"


_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}


class KernelSet:
    """Launchers for activations and weights of one element type."""

    def __init__(self, dtype: torch.dtype):
        if dtype not in _SUFFIX:
            raise KernelError(f"no kernels for {dtype}; supported: float32, bfloat16")
        self.dtype = dtype
        self.suffix = _SUFFIX[dtype]
        self.lib = load_library(self.suffix)
        self._fns: dict[str, object] = {}

    def _fn(self, name):
        fn = self._fns.get(name)
        if fn is None:
            fn = getattr(self.lib, f"sllm_{name}_{self.suffix}")
            fn.restype = c_int
            self._fns[name] = fn
        return fn

    # ------------------------------------------------------------------ embedding
    def embed_rows(self, ids, table, out, err_flag):
        T, d = out.shape
        _check(self._fn("embed_rows")(_ptr(ids, torch.int32, "ids"), _ptr(table, self.dtype, "table"),
                                      _ptr(out, torch.float32, "out"), c_int(T), c_int(d), c_int(table.shape[0]),
                                      _ptr(err_flag, torch.int32, "err"), _stream()), "embed_rows")

    def embed_pair_rows(self, ids, ctx, table, pair_table, buckets, mul_prev, mul_cur, last, out, err_flag):
        """out float32 [T, d] = table[ids[t]] + pair_table[(previous token * mul_prev + ids[t] * mul_cur) mod buckets], the
        pair table's row `buckets` for a sequence's first token; `last` int32 [slots]: the sequences' last tokens (read, then set)."""
        T, d = out.shape
        if tuple(pair_table.shape) != (buckets + 1, d) or table.shape[1] != d or last.dim() != 1:
            raise KernelError(f"embed_pair_rows shapes: table {tuple(table.shape)}, pair table {tuple(pair_table.shape)}, buckets {buckets}")
        _check(self._fn("embed_pair_rows")(_ptr(ids, torch.int32, "ids"), _ptr(ctx.tok_pos, torch.int32, "tok_pos"),
                                           _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(ctx.seq_start, torch.int32, "seq_start"),
                                           _ptr(ctx.slots, torch.int32, "slots"), _ptr(table, self.dtype, "table"),
                                           _ptr(pair_table, self.dtype, "pair_table"), _ptr(out, torch.float32, "out"), c_int(T), c_int(d),
                                           c_int(table.shape[0]), c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur),
                                           _ptr(last, torch.int32, "last"), _ptr(err_flag, torch.int32, "err"), _stream()),
               "embed_pair_rows")

    # ------------------------------------------------------------------ norm
    def add_rmsnorm(self, x, delta, rows, weight, y, eps):
        """x float32 [T,d] residual (+= delta when rows is None); y [n,d] normed output. delta: None,
        [T,d] of this set's dtype, or float32 [P,T,d] partial sums that add up to the addend."""
        d = x.shape[-1]
        n = y.shape[0]
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"norm weight has dtype {weight.dtype}")
        n_parts, stride = 0, 0
        if delta is not None and delta.dim() == 3:
            if delta.dtype != torch.float32 or tuple(delta.shape[1:]) != tuple(x.shape):
                raise KernelError(f"partial sums must be float32 [P, {x.shape[0]}, {d}], found {delta.dtype} {tuple(delta.shape)}")
            n_parts, stride = delta.shape[0], x.shape[0] * d
        elif delta is not None and (delta.dtype != self.dtype or tuple(delta.shape) != tuple(x.shape)):
            raise KernelError(f"addend must be {self.dtype} {tuple(x.shape)}, found {delta.dtype} {tuple(delta.shape)}")
        _check(self._fn("add_rmsnorm")(_ptr(x, torch.float32, "x"), _ptr(delta, None, "delta"), c_int(n_parts),
                                       c_longlong(stride), _ptr(rows, torch.int32, "rows"), _ptr(weight, None, "weight"),
                                       c_int(1 if weight.dtype == torch.float32 else 0), _ptr(y, self.dtype, "y"),
                                       c_int(n), c_int(d), c_float(eps), _stream()), "add_rmsnorm")

    # ------------------------------------------------------------------ matrix products
    def gemm_nt(self, a, w, out):
        """out[M,N] = a[M,K] @ w[N,K]^T; `out` is of this set's dtype or float32. A float32 `out` of
        shape [P,M,N] receives P partial sums (K cut into P parts); the reader adds them."""
        M, K = a.shape
        N = w.shape[0]
        ksplit = out.shape[0] if out.dim() == 3 else 1
        if w.shape[1] != K or tuple(out.shape[-2:]) != (M, N) or (out.dim() == 3 and out.dtype != torch.float32):
            raise KernelError(f"gemm_nt shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
        out_f32 = 1 if (out.dtype == torch.float32 and self.dtype != torch.float32) else 0
        if a.dtype != self.dtype or not a.is_cuda or a.stride(1) != 1:
            raise KernelError(f"gemm_nt: a must be {self.dtype} on a CUDA device with unit column stride")
        _check(self._fn("gemm_nt")(c_void_p(a.data_ptr()), _ptr(w, self.dtype, "w"),
                                   _ptr(out, torch.float32 if out_f32 else self.dtype, "out"), c_int(M), c_int(N),
                                   c_int(K), c_int(a.stride(0)), c_int(w.stride(0)), c_int(N), c_int(out_f32),
                                   c_int(ksplit), _stream()), "gemm_nt")

    @staticmethod
    def gemm_nt_split(m: int, n_out: int, k: int, sm_count: int) -> int:
        """Into how many parts the generic product cuts K when its reader takes partial sums: none for
        up to 8 rows (a block per four columns fills the GPU already) or when the 128-column tiles
        fill it; else enough parts for about two blocks per SM, each at least 256 deep."""
        if m <= 8 or k % 4:
            return 1
        tiles = -(-n_out // 128) * -(-m // (64 if m <= 64 else 128))
        if tiles >= sm_count:
            return 1
        return max(1, min(2 * sm_count // tiles, k // 256, 16))

    # ------------------------------------------------------------------ rotary + cache write
    def rope_kv_write(self, qkv, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv, head_dim, rot,
                      interleaved):
        T, ld = qkv.shape
        _check(self._fn("rope_kv_write")(_ptr(qkv, self.dtype, "qkv"), c_int(ld), _ptr(tok_pos, torch.int32, "tok_pos"),
                                         _ptr(tok_seq, torch.int32, "tok_seq"),
                                         _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                         _ptr(cos_sin, torch.float32, "cos_sin"),
                                         _ptr(kpages, self.dtype if kpages is not None else None, "kpages"),
                                         _ptr(vpages, self.dtype if vpages is not None else None, "vpages"), c_int(T),
                                         c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(rot),
                                         c_int(1 if interleaved else 0), _stream()), "rope_kv_write")

    # ------------------------------------------------------------------ attention
    def attn_paged(self, q, out, seq_start, seq_pos0, block_table, kpages, vpages, n_seqs, max_new, n_heads, n_kv,
                   head_dim, window, scale, softcap=None, sink=None):
        """`softcap`: a score s becomes softcap * tanh(s / softcap) before the softmax; `sink` float32 [n_heads]:
        exp(sink[h]) joins head h's denominator with no key and no value."""
        _check(self._fn("attn_paged")(_ptr(q, self.dtype, "q"), c_int(q.shape[1]), _ptr(out, self.dtype, "out"),
                                      _ptr(seq_start, torch.int32, "seq_start"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
                                      _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                      _ptr(kpages, self.dtype, "kpages"), _ptr(vpages, self.dtype, "vpages"),
                                      c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                      c_int(window or 0), c_float(scale), c_float(softcap or 0.0),
                                      _ptr(sink, torch.float32, "sink"), _stream()), "attn_paged")

    def attn_decode_split(self, q, out, seq_pos0, block_table, kpages, vpages, part, n_seqs, n_heads, n_kv, head_dim,
                          window, scale, n_split, softcap=None, sink=None):
        """One query per sequence, each sequence's keys split over `n_split` blocks (then merged);
        `part`: float32 scratch of n_seqs * n_heads * n_split * (head_dim + 2) elements, or None for one split.
        `softcap`, `sink`: as for `attn_paged`; the sink joins once, where the splits are merged."""
        need = n_seqs * n_heads * n_split * (head_dim + 2) if n_split > 1 else 0
        if need and (part is None or part.numel() < need):
            raise KernelError(f"attn_decode_split scratch holds {0 if part is None else part.numel()} floats, needs {need}")
        _check(self._fn("attn_decode_split")(_ptr(q, self.dtype, "q") if q.is_contiguous() else c_void_p(q.data_ptr()),
                                             c_int(q.stride(0)), _ptr(out, self.dtype, "out"),
                                             _ptr(seq_pos0, torch.int32, "seq_pos0"),
                                             _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
                                             _ptr(kpages, self.dtype, "kpages"), _ptr(vpages, self.dtype, "vpages"),
                                             _ptr(part, torch.float32, "part"), c_int(n_seqs), c_int(n_heads), c_int(n_kv),
                                             c_int(head_dim), c_int(window or 0), c_float(scale), c_int(n_split),
                                             c_float(softcap or 0.0), _ptr(sink, torch.float32, "sink"), _stream()),
               "attn_decode_split")

    @staticmethod
    def attn_decode_split_takes(head_dim: int, q_ld: int) -> bool:
        return head_dim % 4 == 0 and 4 <= head_dim <= 512 and q_ld % 4 == 0

    @staticmethod
    def attn_decode_splits(n_seqs: int, n_heads: int, n_kv: int, pages: int, sm_count: int) -> int:
        """Blocks per (sequence, key/value head, pass over the keys; a pass serves up to four of the
        query heads that share the key/value head): enough for about six blocks of four warps per SM,
        at most one per page."""
        passes = -(-(n_heads // n_kv) // 4)       # (wide heads, above 128: two heads a pass; the estimate stays)
        want = -(-6 * sm_count // max(1, n_seqs * n_kv * passes))
        return max(1, min(want, pages, 64))

    # ------------------------------------------------------------------ feed-forward
    def swiglu(self, gate_up, out, tiled=False):
        T, F = out.shape
        if tuple(gate_up.shape) != (T, 2 * F):
            raise KernelError(f"swiglu shapes: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        _check(self._fn("swiglu")(_ptr(gate_up, self.dtype, "gate_up"), _ptr(out, self.dtype, "out"), c_int(T), c_int(F),
                                  c_int(1 if tiled else 0), _stream()), "swiglu")

    # ------------------------------------------------------------------ fast bfloat16 kernels
    @property
    def tensor_core(self) -> "TensorCoreGemm":
        if self.dtype != torch.bfloat16:
            raise KernelError("the tensor-core GEMM is bfloat16 only")
        if getattr(self, "_tc", None) is None:
            self._tc = TensorCoreGemm()
        return self._tc

    @property
    def prefill_attention_tc(self) -> "PrefillAttentionTC":
        if self.dtype != torch.bfloat16:
            raise KernelError("the tensor-core attention is bfloat16 only")
        if getattr(self, "_fa_tc", None) is None:
            self._fa_tc = PrefillAttentionTC()
        return self._fa_tc

    @property
    def prefill_attention_mma(self) -> "PrefillAttentionMMA":
        k = self.__dict__.get("_prefill_mma")
        if k is None:
            k = self.__dict__["_prefill_mma"] = PrefillAttentionMMA()
        return k

    @property
    def seq(self) -> "SequenceKernels":
        """The kernels of mixers with state along the sequence, for this set's element type."""
        if getattr(self, "_seq", None) is None:
            self._seq = SequenceKernels(self.dtype)
        return self._seq

    @property
    def mix(self) -> "MixKernels":
        """The kernels of latent attention, decayed linear attention, the selective scan, routed experts and
        the norm without statistics, for this set's element type."""
        if getattr(self, "_mix", None) is None:
            self._mix = MixKernels(self.dtype)
        return self._mix

    @property
    def gate(self) -> "GateKernels":
        """The kernels around gated mixers and side inputs (whole-projection query/key norm with the cache write,
        a gate per head, a norm on the way into the stream, a cap on the logits), for this set's element type."""
        if getattr(self, "_gate", None) is None:
            self._gate = GateKernels(self.dtype)
        return self._gate

    @property
    def decode(self) -> "DecodeKernels":
        if self.dtype != torch.bfloat16:
            raise KernelError("the decode kernels are bfloat16 only")
        if getattr(self, "_decode", None) is None:
            self._decode = DecodeKernels()
        return self._decode


class TensorCoreGemm:
    """bfloat16 GEMM on tcgen05 tensor cores with TMA-fed shared memory (the prompt step's products)."""

    def __init__(self):
        self.lib = load_library("gemm_tcgen05")
        for n in ("sllm_gemm_tc_bf16", "sllm_gemm_tc_fold_bf16", "sllm_gemm_tc_skinny_bf16", "sllm_gemm_tc_qkv_rope_bf16",
                  "sllm_gemm_tc_qkv_rope_fold_bf16"):
            getattr(self.lib, n).restype = c_int

    @staticmethod
    def takes(a, w) -> bool:
        return (a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    @staticmethod
    def _owed_args(owed, M):
        if owed is None:
            return c_void_p(None), c_int(0), c_int(0), c_float(0.0)
        sq, width, eps = owed
        if sq.dtype != torch.float32 or sq.dim() != 2 or sq.shape[1] != M or not sq.is_contiguous():
            raise KernelError(f"sums of squares {tuple(sq.shape)} {sq.dtype} for {M} rows")
        return _ptr(sq, torch.float32, "sumsq"), c_int(sq.shape[0]), c_int(width), c_float(eps)

    FOLD_SPAN = 128      # columns to a partial sum of squares that a folded product leaves
    FOLD_MIN_M = 129     # the product that finishes a sublayer for a folded norm runs on the two-SM tiles only
    ONE_SM_FORCED = os.environ.get("SLLM_GEMM_ONE_SM", "0") not in ("", "0")      # a debugging switch of the library

    def gemm(self, a, w, out, err_flag, swiglu=False, owed=None, fold=None):
        """out[M,N] = a @ w^T in bfloat16 or float32; swiglu: out[M,N/2] = silu(gate)*up for w's rows
        tiled 8 gate / 8 up. `err_flag` (int32 on the device) is set if a wait in the kernel timed out.
        `owed` = (sumsq float32 [P, M], width, eps): the rows of `a` are a norm's v * weight whose scale
        rsqrt(sum of v^2 / width + eps) is applied to the output rows instead. `fold` = (norm_weight
        float32 [N], xb bfloat16 [M, N], sumsq_out float32 [ceil(N / 128), M]): `out` is the float32
        residual stream [M, N] (M >= FOLD_MIN_M, N > 128 and a multiple of 32); it receives the product,
        and xb and sumsq_out what the product behind the following norm is owed."""
        M, K = a.shape
        N = w.shape[0]
        if fold is not None:
            norm_w, xb, sq_out = fold
            if (swiglu or out.dtype != torch.float32 or tuple(out.shape) != (M, N) or N % 32 or N <= 128 or M < self.FOLD_MIN_M
                    or tuple(norm_w.shape) != (N,) or norm_w.dtype != torch.float32 or tuple(xb.shape) != (M, N)
                    or xb.dtype != torch.bfloat16 or not xb.is_contiguous() or tuple(sq_out.shape) != (-(-N // self.FOLD_SPAN), M)
                    or not sq_out.is_contiguous() or w.shape[1] != K or out.stride(1) != 1):
                raise KernelError(f"gemm_tc fold: residual {tuple(out.shape)} {out.dtype}, norm weight {tuple(norm_w.shape)}, "
                                  f"xb {tuple(xb.shape)}, sums {tuple(sq_out.shape)} for M={M}, N={N}")
            _check(self.lib.sllm_gemm_tc_fold_bf16(
                c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
                c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1), c_int(2), *self._owed_args(owed, M),
                _ptr(norm_w, torch.float32, "norm_w"), _ptr(xb, torch.bfloat16, "xb"), _ptr(sq_out, torch.float32, "sumsq_out"),
                _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_tc")
            return
        want = (M, N // 2) if swiglu else (M, N)
        if tuple(out.shape) != want or w.shape[1] != K or out.stride(1) != 1:
            raise KernelError(f"gemm_tc shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_tc dtypes: a {a.dtype}, w {w.dtype}, out {out.dtype}")
        if not (a.is_cuda and w.is_cuda and out.is_cuda):
            raise KernelError("gemm_tc runs on a CUDA device only")
        _check(self.lib.sllm_gemm_tc_fold_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
            c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), *self._owed_args(owed, M), c_void_p(None), c_void_p(None), c_void_p(None),
            _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_tc")


    QKV_ROPE_HEAD_DIMS = (64, 128)

    @classmethod
    def rotation_fusable(cls, head_dim: int, rot: int, interleaved: bool) -> bool:
        """Whether the q|k|v product's epilogue can rotate by a (cos, sin) table and fill the cache
        itself: its 32-column chunks must hold whole pairs, or both halves of a fully rotated head."""
        return head_dim in cls.QKV_ROPE_HEAD_DIMS and (interleaved or rot == head_dim)

    def gemm_qkv_rope(self, a, w, qkv, err_flag, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv,
                      head_dim, rot, interleaved, owed=None):
        """qkv[:, :n_heads*head_dim] = rotated queries of a @ w^T (w rows: q | k | v heads); the rotated
        keys and the values go to each row's place in the cache pages and not to `qkv`. `owed`: as in `gemm`."""
        M, K = a.shape
        N = (n_heads + 2 * n_kv) * head_dim
        if tuple(w.shape) != (N, K) or qkv.shape[0] != M or qkv.shape[1] < n_heads * head_dim or qkv.stride(1) != 1:
            raise KernelError(f"gemm_qkv_rope shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16:
            raise KernelError("gemm_qkv_rope works in bfloat16")
        _check(self.lib.sllm_gemm_tc_qkv_rope_fold_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(qkv.data_ptr()), c_int(M), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(qkv.stride(0)), _ptr(tok_pos, torch.int32, "tok_pos"), _ptr(tok_seq, torch.int32, "tok_seq"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), _ptr(cos_sin, torch.float32, "cos_sin"),
            _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"), c_int(n_heads), c_int(n_kv),
            c_int(head_dim), c_int(rot), c_int(1 if interleaved else 0), *self._owed_args(owed, M),
            _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_qkv_rope")

    SKINNY_MAX_M = 128

    ACTS = {None: 0, "gelu_tanh": 1, "relu_squared": 2, "silu": 3}

    def gemm_grouped(self, a, w, out, tile_group, err_flag, act=None, rows_used=None, glu=None):
        """out[M, N] = act(a[M, K] @ w[g]^T) with w [G, N, K] and the 128 rows of `a` from row 128 t on multiplied by
        matrix tile_group[t] (int32 on the device, M / 128 entries): rows laid out so that no 128 hold two groups.
        rows_used: an int32 on the device (one element), how many of the M rows hold anything; the rest is not worked.
        `glu` = (limit, alpha): every matrix's N rows are tiles of 8 gate rows and their 8 up rows, and out [M, N / 2]
        (bfloat16) receives the clamped gate of each pair of sums, g' * sigmoid(alpha g') * (u' + 1); a limit of 0 stands
        for the gate without a clamp, silu(g) * u."""
        M, K = a.shape
        G, N = w.shape[0], w.shape[1]
        if glu is not None and (act is not None or N % 16 or out.dtype != torch.bfloat16 or glu[0] < 0):
            raise KernelError(f"gemm_grouped with a gate: {N} stacked rows a matrix, out {out.dtype}, act {act}, limit {glu[0]}")
        if (w.dim() != 3 or w.shape[2] != K or tuple(out.shape) != (M, N // 2 if glu is not None else N)
                or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
                or out.dtype not in (torch.bfloat16, torch.float32) or tile_group.shape[0] * 128 < M):
            raise KernelError(f"gemm_grouped shapes: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
        fn = self.lib.sllm_gemm_tc_grouped_bf16
        fn.restype = c_int
        _check(fn(_ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(out, None, "out"), c_int(M), c_int(N), c_int(K),
                  c_int(K), c_int(K), c_int(out.shape[1]), c_int(1 if out.dtype == torch.float32 else 0),
                  _ptr(tile_group, torch.int32, "tile_group"), c_int(G), c_int(self.ACTS[act]), _ptr(rows_used, torch.int32, "rows_used"),
                  c_int(0 if glu is None else 1), c_float(0.0 if glu is None else glu[0]), c_float(0.0 if glu is None else glu[1]),
                  _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_grouped")

    def gemm_act(self, a, w, out, err_flag, act: str):
        """out[M, N] = act(a @ w^T): the activation on the float sums, in the product's epilogue."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N) or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_act shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
        fn = self.lib.sllm_gemm_tc_act_bf16
        fn.restype = c_int
        _check(fn(c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
                  c_int(a.stride(0)), c_int(w.stride(0)), c_int(N), c_int(1 if out.dtype == torch.float32 else 0), c_int(self.ACTS[act]),
                  _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_act")

    def gemm_skinny(self, a, w, out, err_flag, swiglu=False):
        """The same product for at most 128 rows of `a`, with the weights as the tensor cores' 128-row
        operand and a grid over (128 weight rows, K splits). out [M,N] bfloat16 or float32, or
        [M,N/2] with swiglu; float32 [P,M,N]: K split P ways, out receives the partial sums."""
        M, K = a.shape
        N = w.shape[0]
        ksplit = out.shape[0] if out.dim() == 3 else 1
        want = (M, N // 2) if swiglu else ((ksplit, M, N) if out.dim() == 3 else (M, N))
        if out.dim() == 3 and out.dtype != torch.float32:
            raise KernelError("partial sums are written in float32")
        if tuple(out.shape) != want or w.shape[1] != K or not out.is_contiguous():
            raise KernelError(f"gemm_skinny shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_skinny dtypes: a {a.dtype}, w {w.dtype}, out {out.dtype}")
        if not (a.is_cuda and w.is_cuda and out.is_cuda):
            raise KernelError("gemm_skinny runs on a CUDA device only")
        _check(self.lib.sllm_gemm_tc_skinny_bf16(
            c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
            c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), c_int(ksplit), _ptr(err_flag, torch.int32, "err_flag"), _stream()), "gemm_skinny")

    def prefers_skinny(self, a, w, kind: str, sm_count: int) -> bool:
        """True where the few-rows kernel is the fastest of the three products for a [M,K] x [N,K]^T
        (measured on the layer shapes of 1-8 B models): 9..128 rows; always when the reader takes
        partial sums ("partials": K is split to fill the GPU); with the SiLU gate ("swiglu") up to 64
        rows; a plain product ("plain") from 33 rows on and only while its N/128 blocks fit one wave
        of the GPU's `sm_count` SMs."""
        M, N = a.shape[0], w.shape[0]
        if not (8 < M <= self.SKINNY_MAX_M and self.takes(a, w)):
            return False
        if kind == "partials":
            return True
        if kind == "swiglu":
            return M <= 64
        return M > 32 and N <= 128 * sm_count

    @staticmethod
    def skinny_split(n_out: int, k: int, sm_count: int) -> int:
        """Over how many blocks to split K so that the (n_out / 128) x split grid about fills the GPU."""
        tiles = -(-n_out // 128)
        return max(1, min(sm_count // tiles, k // 256, 16))


class PrefillAttentionTC:
    """tcgen05 causal attention of a prompt step over the paged cache (bfloat16, head width 64 or 128)."""
    HEAD_DIMS = (64, 128)

    def __init__(self):
        self.lib = load_library("attn_prefill_tcgen05")
        self.lib.sllm_attn_prefill_tc_bf16.restype = c_int

    def attn(self, q, out, seq_start, seq_pos0, block_table, kpages, vpages, n_seqs, max_new, n_heads, n_kv, head_dim,
             window, scale, err_flag, softcap=None, sink=None):
        """`softcap`: a score s becomes softcap * tanh(s / softcap) before the softmax; `sink` float32 [n_heads]: exp(sink[h])
        joins head h's denominator with no key and no value."""
        _check(self.lib.sllm_attn_prefill_tc_bf16(
            _ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), c_int(q.shape[0]), _ptr(out, torch.bfloat16, "out"),
            _ptr(seq_start, torch.int32, "seq_start"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
            _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"), c_longlong(kpages.shape[0]),
            c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale),
            c_float(softcap or 0.0), _ptr(sink, torch.float32, "sink"), _ptr(err_flag, torch.int32, "err_flag"), _stream()),
            "attn_prefill_tc")


class PrefillAttentionMMA:
    """Causal attention of a prompt step on mma.sync for key and value widths the tcgen05 kernels do not take (bfloat16): keys
    of 64, 96, 128, 192 or 256, values of 64 or 128; rows in storage may be wider than what is used."""
    KEY_WIDTHS = (64, 96, 128, 192, 256)
    VALUE_WIDTHS = (64, 128)

    def __init__(self):
        self.lib = load_library("attn_prefill_mma")
        self.lib.sllm_attn_prefill_mma_bf16.restype = c_int

    @classmethod
    def widths_for(cls, key_dim: int, value_dim: int):
        """The (key width, value width) the kernel would run for heads of these widths (padded with zeros), or None."""
        k = next((w for w in cls.KEY_WIDTHS if w >= key_dim), None)
        v = next((w for w in cls.VALUE_WIDTHS if w >= value_dim), None)
        return None if k is None or v is None else (k, v)

    def attn(self, q, q_hw, out, o_hw, seq_start, seq_pos0, block_table, kpages, vpages, n_seqs, max_new, n_heads, n_kv, kd, vd,
             window, scale, softcap=None, sink=None):
        """q [T, n_heads * q_hw], out [T, n_heads * o_hw] (the o_hw - vd columns past a head's values are set to 0), kpages
        [pages, n_kv, 64, k_w], vpages [pages, n_kv, 64, v_w]; kd and vd are the widths used."""
        _check(self.lib.sllm_attn_prefill_mma_bf16(
            _ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), c_int(q_hw), _ptr(out, torch.bfloat16, "out"), c_int(out.shape[1]),
            c_int(o_hw), _ptr(seq_start, torch.int32, "seq_start"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"),
            c_int(kpages.shape[-1]), _ptr(vpages, torch.bfloat16, "vpages"), c_int(vpages.shape[-1]), c_int(n_seqs), c_int(max_new),
            c_int(n_heads), c_int(n_kv), c_int(kd), c_int(vd), c_int(window or 0), c_float(scale), c_float(softcap or 0.0),
            _ptr(sink, torch.float32, "sink"), _stream()), "attn_prefill_mma")


class DecodeKernels:
    """Weight-streaming small-M product and split-key attention for the bfloat16 decode step."""
    HEAD_DIMS = (16, 32, 64, 128, 256)
    MAX_M = 64

    def __init__(self):
        self.lib = load_library("decode_bf16")
        for n in ("sllm_gemm_small_m_bf16", "sllm_gemm_small_m_fold_bf16", "sllm_attn_decode_bf16",
                  "sllm_attn_decode_merged_bf16", "sllm_attn_decode_rope_bf16", "sllm_attn_decode_capped_bf16"):
            getattr(self.lib, n).restype = c_int
        self.lib.sllm_attn_decode_scratch_bytes.restype = c_longlong
        self.lib.sllm_attn_decode_uses_mma.restype = c_int

    @staticmethod
    def takes(a, w) -> bool:
        K = a.shape[1]
        return (a.shape[0] <= DecodeKernels.MAX_M and K % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)

    @staticmethod
    def prefers(a, w, sm_count: int) -> bool:
        """True when this kernel is the faster one for the shape: always up to 16 rows; beyond that
        only while the output is too narrow to give the 128 x 256 tensor-core tiles enough blocks
        (fewer than a third of the SMs; measured at 148: 48 tiles)."""
        return DecodeKernels.takes(a, w) and (a.shape[0] <= 16 or 3 * -(-w.shape[0] // 256) <= sm_count)

    @staticmethod
    def rotation_fusable(rot: int, interleaved: bool) -> bool:
        """Whether the decode attention kernel can rotate queries and the new key by a (cos, sin)
        table itself: its 16-byte vectors must not straddle the rotary width or its half."""
        return rot >= 2 and rot % (8 if interleaved else 16) == 0

    MAX_SPLITS = 64      # beyond this the merging block falls back to a slow loop

    def attention_splits(self, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, pages: int, sm_count: int) -> int:
        """Over how many blocks a decode step splits each sequence's keys: about as many blocks as are
        resident at once (a second wave that is far from full costs a whole one), never more than the
        longest sequence has pages. The tensor-core kernel (grouped queries, or very few sequences)
        has fatter blocks: its registers allow four per SM at width 64, two at width 128, and it wants
        at least four pages each. The one-head kernel is built for seven per SM (three where it serves
        several query heads per key/value head at other widths); a tenth more blocks than that still
        beat leaving a quarter of the places empty (measured at context 4,096: 12 sequences 64.5 us
        with 1,152 blocks against 74.6 with 768; 6 sequences 36.1 with 1,152 against 37.2 with 960;
        16 sequences 84.6 with 1,024 against 98.8 with 1,536)."""
        pairs = max(1, n_seqs * n_kv_heads)
        if self.lib.sllm_attn_decode_uses_mma(c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim)):
            want, cap = ((4 if head_dim <= 64 else 2) * sm_count) // pairs, max(1, pages // 4)
        else:
            want, cap = ((39 if n_heads == n_kv_heads else 17) * sm_count) // (5 * pairs), pages
        n = max(1, min(want, cap, DecodeKernels.MAX_SPLITS))
        per = -(-pages // n)                   # pages a block takes; the fewest blocks that need no more each
        return max(1, -(-pages // per)) if pages > 0 else n

    FOLD_MAX_M = 16      # rows up to which a product can take over one half of a norm

    def gemm_small_m(self, a, w, out, swiglu=False, owed=None, fold=None):
        """out[M,N] = a @ w^T (bfloat16 or float32 out); swiglu: out[M,N/2] = silu(gate)*up for w rows
        tiled 8 gate / 8 up; out float32 [P,M,N]: K split P ways, out receives the partial sums.
        `owed` = (sumsq float32 [P, M], width, eps): the rows of `a` are a norm's v * weight whose scale
        rsqrt(sum of v^2 / width + eps) is applied to the output rows instead. `fold` = (norm_weight
        float32 [N], xb bfloat16 [M, N], sumsq_out float32 [ceil(N / 16), M]): `out` is the float32
        residual stream [M, N]; it receives the product, and xb and sumsq_out what the product after
        the following norm is owed (M <= FOLD_MAX_M)."""
        M, K = a.shape
        N = w.shape[0]
        if owed is not None or fold is not None:
            return self._gemm_small_m_fold(a, w, out, swiglu, owed, fold)
        ksplit = out.shape[0] if out.dim() == 3 else 1
        want = (M, N // 2) if swiglu else ((ksplit, M, N) if out.dim() == 3 else (M, N))
        if out.dim() == 3 and out.dtype != torch.float32:
            raise KernelError("partial sums are written in float32")
        if tuple(out.shape) != want or w.shape[1] != K:
            raise KernelError(f"gemm_small_m shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_small_m output dtype {out.dtype}")
        _check(self.lib.sllm_gemm_small_m_bf16(
            _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else c_void_p(a.data_ptr()),
            _ptr(w, torch.bfloat16, "w"), _ptr(out, None, "out"), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(1 if swiglu else 0), c_int(ksplit), _stream()), "gemm_small_m")

    def _gemm_small_m_fold(self, a, w, out, swiglu, owed, fold):
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.dim() != 2 or (fold is not None and swiglu):
            raise KernelError(f"gemm_small_m shapes: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        sumsq_in, n_in, width, eps = c_void_p(None), 0, 0, 0.0
        if owed is not None:
            sq, width, eps = owed
            if sq.dtype != torch.float32 or sq.dim() != 2 or sq.shape[1] != M or not sq.is_contiguous():
                raise KernelError(f"gemm_small_m: sums of squares {tuple(sq.shape)} {sq.dtype} for {M} rows")
            sumsq_in, n_in = _ptr(sq, torch.float32, "sumsq"), sq.shape[0]
        if fold is not None:
            norm_w, xb, sq_out = fold
            tiles = -(-N // 16)
            if (M > self.FOLD_MAX_M or out.dtype != torch.float32 or tuple(out.shape) != (M, N) or tuple(norm_w.shape) != (N,)
                    or tuple(xb.shape) != (M, N) or not xb.is_contiguous() or tuple(sq_out.shape) != (tiles, M)
                    or not sq_out.is_contiguous()):
                raise KernelError(f"gemm_small_m fold: residual {tuple(out.shape)} {out.dtype}, norm weight {tuple(norm_w.shape)}, "
                                  f"xb {tuple(xb.shape)}, sums {tuple(sq_out.shape)} for M={M}, N={N}")
            tail = (_ptr(norm_w, torch.float32, "norm_w"), _ptr(xb, torch.bfloat16, "xb"), _ptr(sq_out, torch.float32, "sumsq_out"))
            epilogue = 2
        else:
            want = (M, N // 2) if swiglu else (M, N)
            if tuple(out.shape) != want or out.dtype not in (torch.bfloat16, torch.float32):
                raise KernelError(f"gemm_small_m out {tuple(out.shape)} {out.dtype}, want {want}")
            tail = (c_void_p(None), c_void_p(None), c_void_p(None))
            epilogue = 1 if swiglu else 0
        _check(self.lib.sllm_gemm_small_m_fold_bf16(
            _ptr(a, torch.bfloat16, "a") if a.is_contiguous() else c_void_p(a.data_ptr()),
            _ptr(w, torch.bfloat16, "w"), _ptr(out, None, "out"), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
            c_int(w.stride(0)), c_int(out.stride(-2)), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(epilogue), c_int(1), sumsq_in, c_int(n_in), c_int(width), c_float(eps), *tail, _stream()), "gemm_small_m")

    def attn_decode_rope(self, qkv, out, seq_pos0, block_table, kpages, vpages, scratch, tickets, cos_sin, rot,
                         interleaved, write_kv, n_seqs, n_heads, n_kv, head_dim, window, scale, n_split):
        """Rotary positions, cache write and attention of a decode step in one kernel: `qkv` holds the
        unrotated [q | k | v] rows of the step (only q when write_kv is false)."""
        need = self.lib.sllm_attn_decode_scratch_bytes(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_split))
        if scratch.numel() * scratch.element_size() < need or tickets.numel() < n_seqs * n_kv:
            raise KernelError("attn_decode_rope: scratch or tickets too small")
        width = (n_heads + 2 * n_kv) * head_dim if write_kv else n_heads * head_dim
        if qkv.shape[1] < width:
            raise KernelError(f"attn_decode_rope: rows of {qkv.shape[1]} columns, need {width}")
        _check(self.lib.sllm_attn_decode_rope_bf16(
            _ptr(qkv, torch.bfloat16, "qkv"), c_int(qkv.shape[1]), _ptr(out, torch.bfloat16, "out"),
            _ptr(seq_pos0, torch.int32, "seq_pos0"), _ptr(block_table, torch.int32, "block_table"),
            c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"),
            _ptr(scratch, torch.float32, "scratch"), _ptr(tickets, torch.int32, "tickets"),
            _ptr(cos_sin, torch.float32, "cos_sin"), c_int(rot), c_int(1 if interleaved else 0), c_int(1 if write_kv else 0),
            c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale), c_int(n_split),
            _stream()), "attn_decode_rope")

    def split_for(self, n_out: int, k: int, sm_count: int) -> int:
        """Over how many blocks to split K so that a product with few output rows still fills the GPU."""
        tiles = -(-n_out // 16)
        return max(1, min(8, (4 * sm_count) // tiles, k // 512))

    def attn_decode(self, q, out, seq_pos0, block_table, kpages, vpages, scratch, n_seqs, n_heads, n_kv, head_dim,
                    window, scale, n_split, tickets=None):
        """`tickets` (int32 [>= n_seqs * n_kv], zero before its first use, left zero): the last split
        to finish merges the partial results in the same kernel; without it a second kernel merges."""
        need = self.lib.sllm_attn_decode_scratch_bytes(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_split))
        if scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attn_decode scratch holds {scratch.numel() * scratch.element_size()} bytes, needs {need}")
        head = (_ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), _ptr(out, torch.bfloat16, "out"),
                _ptr(seq_pos0, torch.int32, "seq_pos0"), _ptr(block_table, torch.int32, "block_table"),
                c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"), _ptr(vpages, torch.bfloat16, "vpages"),
                _ptr(scratch, torch.float32, "scratch"))
        tail = (c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale),
                c_int(n_split), _stream())
        if tickets is None:
            _check(self.lib.sllm_attn_decode_bf16(*head, *tail), "attn_decode")
        else:
            if tickets.numel() < n_seqs * n_kv:
                raise KernelError(f"attn_decode tickets hold {tickets.numel()} ints, needs {n_seqs * n_kv}")
            _check(self.lib.sllm_attn_decode_merged_bf16(*head, _ptr(tickets, torch.int32, "tickets"), *tail), "attn_decode")


    def uses_tensor_cores(self, n_seqs: int, n_heads: int, n_kv: int, head_dim: int) -> bool:
        """Whether decode attention of this shape runs on the kernel that puts a group's query heads on the tensor cores
        (the one that knows capped scores and sinks)."""
        return bool(self.lib.sllm_attn_decode_uses_mma(c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim))) \
            and not os.environ.get("SLLM_DECODE_SCALAR")

    def attn_decode_capped(self, q, out, seq_pos0, block_table, kpages, vpages, scratch, tickets, n_seqs, n_heads, n_kv, head_dim,
                           window, scale, n_split, softcap=None, sink=None):
        """`attn_decode` with tickets where a score s becomes softcap * tanh(s / softcap) and exp(sink[h]) (float32
        [n_heads]) joins head h's denominator once; only for shapes `uses_tensor_cores` answers."""
        need = self.lib.sllm_attn_decode_scratch_bytes(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_split))
        if scratch.numel() * scratch.element_size() < need or tickets.numel() < n_seqs * n_kv:
            raise KernelError(f"attn_decode_capped scratch holds {scratch.numel() * scratch.element_size()} bytes, needs {need}")
        _check(self.lib.sllm_attn_decode_capped_bf16(
            _ptr(q, torch.bfloat16, "q"), c_int(q.shape[1]), _ptr(out, torch.bfloat16, "out"), _ptr(seq_pos0, torch.int32, "seq_pos0"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), _ptr(kpages, torch.bfloat16, "kpages"),
            _ptr(vpages, torch.bfloat16, "vpages"), _ptr(scratch, torch.float32, "scratch"), _ptr(tickets, torch.int32, "tickets"),
            c_int(n_seqs), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(window or 0), c_float(scale), c_int(n_split),
            c_float(softcap or 0.0), _ptr(sink, torch.float32, "sink"), _stream()), "attn_decode_capped")


class SequenceKernels:
    """Launchers of sequence_kernels.cuh: the norm with weighted addends, the short causal convolution
    with state, the cache write with value norm, attention with values wider or narrower than keys,
    the gated delta rule and the gated linear recurrence. `dtype` is the element type of activations
    and weights; state, sums and gates are float32 in both sets."""
    MAX_ADDENDS = 16

    def __init__(self, dtype: torch.dtype):
        if dtype not in _SUFFIX:
            raise KernelError(f"no kernels for {dtype}; supported: float32, bfloat16")
        self.dtype, self.suffix = dtype, _SUFFIX[dtype]
        self.lib = load_library("seq_" + self.suffix)
        self._fns: dict[str, object] = {}

    def _fn(self, name):
        fn = self._fns.get(name)
        if fn is None:
            fn = getattr(self.lib, f"sllm_{name}_{self.suffix}")
            fn.restype = c_int
            self._fns[name] = fn
        return fn

    def _flag(self, t, name):
        """1 for a float32 buffer, 0 for one of the element type."""
        if t.dtype == torch.float32:
            return 1
        if t.dtype != self.dtype:
            raise KernelError(f"{name} has dtype {t.dtype}; expected float32 or {self.dtype}")
        return 0

    @staticmethod
    def _view(t, name):
        """Pointer of a [rows, columns] buffer whose rows may be strided (a column slice)."""
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{name} must be a CUDA tensor [rows, columns] with unit column stride")
        return c_void_p(t.data_ptr())

    def add_norm(self, x, addends, rows, weight, y, eps, center):
        """x float32 [T, d] += sum coef * addend (when rows is None); y [n, d] (float32 or element type) the
        norm of the (chosen) rows: (v - mean) / sqrt(var + eps) * w if `center`, else v / sqrt(mean v^2 + eps) * w.
        `addends`: list of (tensor [T, d] float32 or element type, coefficient)."""
        d = x.shape[-1]
        if len(addends) > self.MAX_ADDENDS:
            raise KernelError(f"add_norm takes at most {self.MAX_ADDENDS} addends, got {len(addends)}")
        for t, _ in addends:
            if tuple(t.shape) != tuple(x.shape) or not t.is_contiguous():
                raise KernelError(f"addend {tuple(t.shape)} does not fit the stream {tuple(x.shape)}")
        n = len(addends)
        ptrs = (c_void_p * max(1, n))(*[t.data_ptr() for t, _ in addends])
        coefs = (c_float * max(1, n))(*[float(c) for _, c in addends])
        flags = (c_int * max(1, n))(*[self._flag(t, "addend") for t, _ in addends])
        _check(self._fn("add_norm")(_ptr(x, torch.float32, "x"), ptrs, coefs, flags, c_int(n), _ptr(rows, torch.int32, "rows"),
                                    _ptr(weight, None, "weight"), c_int(self._flag(weight, "weight")),
                                    _ptr(y, None, "y"), c_int(self._flag(y, "y")), c_int(y.shape[0]), c_int(d), c_float(eps),
                                    c_int(1 if center else 0), _stream()), "add_norm")

    def causal_conv(self, x, weight, state, ctx, y, taps, in_bias=None, out_bias=None, add_input=False, act=None, y2=None):
        """y[t] = act(sum_j weight[:, j] * in(t - taps + 1 + j) + out_bias (+ in(t))), in = x + in_bias, over the
        rows of each sequence of the step; rows before the step come from `state` float32 [slots, taps - 1, C],
        which afterwards holds the sequence's last taps - 1 inputs. x, y: [T, C] views, float32 or element type."""
        T, C = x.shape
        if tuple(weight.shape) != (C, taps) or tuple(y.shape) != (T, C) or (taps > 1 and tuple(state.shape[1:]) != (taps - 1, C)):
            raise KernelError(f"causal_conv shapes: x {tuple(x.shape)}, weight {tuple(weight.shape)}, y {tuple(y.shape)}")
        b_f32 = 0
        for b in (in_bias, out_bias):
            if b is not None:
                b_f32 = self._flag(b, "bias")
        _check(self._fn("causal_conv")(
            self._view(x, "x"), c_int(self._flag(x, "x")), c_int(x.stride(0)), _ptr(weight, None, "weight"),
            c_int(self._flag(weight, "weight")), _ptr(in_bias, None, "in_bias"), _ptr(out_bias, None, "out_bias"), c_int(b_f32),
            _ptr(state, torch.float32, "state") if taps > 1 else c_void_p(0), _ptr(ctx.seq_start, torch.int32, "seq_start"),
            _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(ctx.slots, torch.int32, "slots"), self._view(y, "y"),
            c_int(self._flag(y, "y")), c_int(y.stride(0)), self._view(y2, "y2") if y2 is not None else c_void_p(0),
            c_int(y2.stride(0) if y2 is not None else 0), c_int(T), c_int(ctx.n_seqs), c_int(C), c_int(taps),
            c_int(1 if add_input else 0), c_int({None: 0, "silu": 1}[act]), _stream()), "causal_conv")

    def kv_store(self, qkv, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv, head_dim, v_dim, rot,
                 interleaved, v_eps):
        """Rotate queries (in place) and keys by the table, store keys and values (divided by their root
        mean square when v_eps is not None) at the rows' places in the cache pages."""
        T, ld = qkv.shape
        _check(self._fn("kv_store")(_ptr(qkv, self.dtype, "qkv"), c_int(ld), _ptr(tok_pos, torch.int32, "tok_pos"),
                                    _ptr(tok_seq, torch.int32, "tok_seq"), _ptr(block_table, torch.int32, "block_table"),
                                    c_int(block_table.shape[1]), _ptr(cos_sin, torch.float32, "cos_sin"),
                                    _ptr(kpages, self.dtype if kpages is not None else None, "kpages"),
                                    _ptr(vpages, self.dtype if vpages is not None else None, "vpages"), c_int(T), c_int(n_heads),
                                    c_int(n_kv), c_int(head_dim), c_int(v_dim), c_int(rot), c_int(1 if interleaved else 0),
                                    c_float(-1.0 if v_eps is None else v_eps), _stream()), "kv_store")

    def attn_wide_value(self, q, out, tok_pos, tok_seq, block_table, kpages, vpages, n_heads, n_kv, head_dim, v_dim, window, scale):
        _check(self._fn("attn_wide_value")(_ptr(q, self.dtype, "q"), c_int(q.shape[1]), _ptr(out, self.dtype, "out"),
                                           c_int(out.shape[1]), _ptr(tok_pos, torch.int32, "tok_pos"),
                                           _ptr(tok_seq, torch.int32, "tok_seq"), _ptr(block_table, torch.int32, "block_table"),
                                           c_int(block_table.shape[1]), _ptr(kpages, self.dtype, "kpages"),
                                           _ptr(vpages, self.dtype, "vpages"), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv),
                                           c_int(head_dim), c_int(v_dim), c_int(window or 0), c_float(scale), _stream()),
               "attn_wide_value")

    def delta_prepare(self, qk, ba, a_log, dt_bias, bd, n_heads, n_kv, dk):
        """qk float32 rows [G dk | G dk]: queries and keys become unit vectors (queries times dk^-1/2) in place;
        bd float32 [T, 2H + G] receives beta = sigmoid(ba[:, :H]), decay = exp(-exp(a_log) softplus(ba[:, H:2H] +
        dt_bias)) and k . q per query/key head."""
        if tuple(bd.shape) != (qk.shape[0], 2 * n_heads + n_kv):
            raise KernelError(f"delta_prepare: bd is {tuple(bd.shape)}, expected {(qk.shape[0], 2 * n_heads + n_kv)}")
        _check(self._fn("delta_prepare")(self._view(qk, "qk"), c_int(qk.stride(0)), self._view(ba, "ba"), c_int(ba.stride(0)),
                                         _ptr(a_log, None, "a_log"), _ptr(dt_bias, None, "dt_bias"),
                                         c_int(self._flag(a_log, "a_log")), _ptr(bd, torch.float32, "bd"), c_int(qk.shape[0]),
                                         c_int(n_heads), c_int(n_kv), c_int(dk), _stream()), "delta_prepare")

    def delta_rule(self, qk, v, bd, state, ctx, o, n_heads, n_kv, dk, dv):
        """qk float32 rows [G dk queries | G dk keys] (unit vectors), v float32 [T, H dv], bd float32 [T, 2H + G]
        (beta | decay | k . q, as `delta_prepare` leaves them), state float32 [slots, H, dk, dv] (read and
        advanced), o float32 [T, H dv]."""
        if tuple(bd.shape) != (qk.shape[0], 2 * n_heads + n_kv):
            raise KernelError(f"delta_rule: bd is {tuple(bd.shape)}, expected {(qk.shape[0], 2 * n_heads + n_kv)}")
        if qk.dtype != torch.float32 or v.dtype != torch.float32 or tuple(state.shape[1:]) != (n_heads, dk, dv):
            raise KernelError("delta_rule works on float32 queries, keys, values and state [slots, heads, dk, dv]")
        _check(self._fn("delta_rule")(self._view(qk, "qk"), c_int(qk.stride(0)), self._view(v, "v"), c_int(v.stride(0)),
                                      _ptr(bd, torch.float32, "bd"), _ptr(state, torch.float32, "state"),
                                      _ptr(ctx.seq_start, torch.int32, "seq_start"), _ptr(ctx.slots, torch.int32, "slots"),
                                      _ptr(o, torch.float32, "o"), c_int(ctx.n_seqs), c_int(max(1, ctx.max_new)), c_int(n_heads),
                                      c_int(n_kv), c_int(dk), c_int(dv), _stream()), "delta_rule")

    def gated_unit_rms(self, o, gate, weight, y, n_heads, dv, eps):
        _check(self._fn("gated_unit_rms")(_ptr(o, torch.float32, "o"), self._view(gate, "gate"), c_int(gate.stride(0)),
                                          _ptr(weight, None, "weight"), c_int(self._flag(weight, "weight")),
                                          _ptr(y, self.dtype, "y"), c_int(o.shape[0]), c_int(n_heads), c_int(dv), c_float(eps),
                                          _stream()), "gated_unit_rms")

    SCAN_WALK_MAX = 4     # rows of a sequence in one step up to which a thread walks them one after the other

    def rglru_scan(self, gates, u, yraw, ra_b, ri_b, lam, y_b, state, ctx, out, block_size):
        """gates float32 [blocks, T, 2 * block_size], u float32 [T, W], yraw [T, W] view of the element type,
        state float32 [slots, W] (read and advanced), out [T, W] of the element type."""
        T, W = u.shape
        if gates.dtype != torch.float32 or tuple(gates.shape) != (W // block_size, T, 2 * block_size) or yraw.dtype != self.dtype:
            raise KernelError(f"rglru_scan shapes: gates {tuple(gates.shape)} {gates.dtype}, u {tuple(u.shape)}")
        scratch = None
        if ctx.max_new > self.SCAN_WALK_MAX:        # a long portion: the scan runs in pieces, which need room for their ends
            piece = self._fn("rglru_piece_rows")()
            scratch = torch.empty((2 * ctx.n_seqs * -(-ctx.max_new // piece) * W,), dtype=torch.float32, device=u.device)
        _check(self._fn("rglru_scan")(_ptr(gates, torch.float32, "gates"), _ptr(u, torch.float32, "u"), self._view(yraw, "yraw"),
                                      c_int(yraw.stride(0)), _ptr(ra_b, None, "ra_b"), _ptr(ri_b, None, "ri_b"),
                                      _ptr(lam, None, "lam"), _ptr(y_b, None, "y_b"), c_int(self._flag(lam, "lam")),
                                      _ptr(state, torch.float32, "state"), _ptr(ctx.seq_start, torch.int32, "seq_start"),
                                      _ptr(ctx.slots, torch.int32, "slots"), _ptr(out, self.dtype, "out"),
                                      _ptr(scratch, torch.float32, "scratch"), c_int(max(1, ctx.max_new)), c_int(T),
                                      c_int(ctx.n_seqs), c_int(W), c_int(block_size), _stream()), "rglru_scan")


class MixKernels:
    """Launchers of mix_kernels.cuh: the norm without statistics fused with the residual sum, activations in
    place, linear attention with a decay per head, the gated read-out norm over a row, attention over a cached
    latent (store, absorb, scores and sums, expand), the selective scan, and routed experts (router, pairs one
    by one, pairs grouped by expert). `dtype` is the element type of activations and weights; state, sums,
    scores and gates are float32 in both sets."""
    ACTS = {"gelu_tanh": 1, "relu_squared": 2, "silu": 3}
    GATES = {"sigmoid": 1, "silu": 2}

    def __init__(self, dtype: torch.dtype):
        if dtype not in _SUFFIX:
            raise KernelError(f"no kernels for {dtype}; supported: float32, bfloat16")
        self.dtype, self.suffix = dtype, _SUFFIX[dtype]
        self.lib = load_library("mix_" + self.suffix)
        self._fns: dict[str, object] = {}

    _fn = SequenceKernels._fn
    _flag = SequenceKernels._flag
    _view = staticmethod(SequenceKernels._view)

    def dyt_add_norm(self, x, addend, post, rows, weight, bias, alpha, out):
        """v = x[row] + a, a = the addend ([T, d] of the element type or float32, or float32 [P, T, d] partial
        sums; None: nothing) passed through tanh(pa * a) * pw + pb when `post` = (pw, pb, pa) is given; x is
        updated in place when rows is None. out[r] = tanh(alpha * v) * weight + bias. weight, bias, pw, pb float32."""
        T, d = x.shape
        n_parts, stride, y_f32 = 0, 0, 0
        if addend is not None:
            if tuple(addend.shape[-2:]) != (T, d) or (addend.dim() == 3 and addend.dtype != torch.float32):
                raise KernelError(f"addend {tuple(addend.shape)} {addend.dtype} does not fit the stream {tuple(x.shape)}")
            n_parts, stride = (addend.shape[0], T * d) if addend.dim() == 3 else (1, 0)
            y_f32 = self._flag(addend, "addend")
        pw, pb, pa = post if post is not None else (None, None, 0.0)
        _check(self._fn("dyt_add_norm")(
            _ptr(x, torch.float32, "x"), _ptr(addend, None, "addend"), c_int(y_f32), c_int(n_parts), c_longlong(stride),
            _ptr(pw, torch.float32, "post weight"), _ptr(pb, torch.float32, "post bias"), c_float(pa),
            c_int(1 if post is not None else 0), c_int(1), _ptr(rows, torch.int32, "rows"), _ptr(weight, torch.float32, "weight"),
            _ptr(bias, torch.float32, "bias"), c_float(alpha), c_int(1), _ptr(out, None, "out"), c_int(self._flag(out, "out")),
            c_int(out.shape[0]), c_int(d), _stream()), "dyt_add_norm")

    def act_inplace(self, x, kind: str):
        _check(self._fn("act_inplace")(_ptr(x, self.dtype, "x"), c_longlong(x.numel()), c_int(self.ACTS[kind]), _stream()),
               "act_inplace")

    def lin_attn_decay(self, proj, q_col, k_col, v_col, decay, state, ctx, o, n_heads, dk, dv):
        """proj [T, ld] of the element type holding the raw q, k, v projections at the given columns (SiLU is
        applied on reading); decay float32 [H]; state float32 [slots, H, dk, dv] (read and advanced); o float32 [T, H dv]."""
        if tuple(state.shape[1:]) != (n_heads, dk, dv) or tuple(o.shape) != (proj.shape[0], n_heads * dv):
            raise KernelError(f"lin_attn_decay shapes: state {tuple(state.shape)}, o {tuple(o.shape)}")
        _check(self._fn("lin_attn_decay")(
            _ptr(proj, self.dtype, "proj"), c_int(proj.shape[1]), c_int(q_col), c_int(k_col), c_int(v_col),
            _ptr(decay, torch.float32, "decay"), _ptr(state, torch.float32, "state"), _ptr(ctx.seq_start, torch.int32, "seq_start"),
            _ptr(ctx.slots, torch.int32, "slots"), _ptr(o, torch.float32, "o"), c_int(ctx.n_seqs), c_int(max(1, ctx.max_new)),
            c_int(n_heads), c_int(dk), c_int(dv), c_int(ctx.engine.sm_count), _stream()), "lin_attn_decay")

    def gated_row_rms(self, o, gate, weight, y, eps, gate_act: str):
        _check(self._fn("gated_row_rms")(_ptr(o, torch.float32, "o"), self._view(gate, "gate"), c_int(gate.stride(0)),
                                         _ptr(weight, torch.float32, "weight"), c_int(1), _ptr(y, self.dtype, "y"),
                                         c_int(o.shape[0]), c_int(o.shape[1]), c_float(eps), c_int(self.GATES[gate_act]), _stream()),
               "gated_row_rms")

    def latent_store(self, q, n_heads, dim, dkv, norm_w, eps, cos_sin, rot, ctx, block_table, pages, rank, rot_dim, half=False):
        """Rotates the last rot_dim dims of every query head of q [T, H (dim + rot_dim)] in place (pairs of neighbours, or
        with `half` dim i with dim i + rot / 2) and, with
        `pages`, stores [dkv[:rank] / rms * norm_w | rotated dkv[rank:]] at the rows' places. q and dkv may be
        column slices of one buffer."""
        _check(self._fn("latent_store")(
            self._view(q, "q"), c_int(q.stride(0)), c_int(n_heads), c_int(dim),
            self._view(dkv, "dkv") if dkv is not None else c_void_p(0), c_int(dkv.stride(0) if dkv is not None else 0),
            _ptr(norm_w, torch.float32, "norm weight"), c_int(1), c_float(eps),
            _ptr(cos_sin, torch.float32, "cos_sin"), c_int(rot), c_int(1 if half else 0), _ptr(ctx.tok_pos, torch.int32, "tok_pos"),
            _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
            _ptr(pages, self.dtype if pages is not None else None, "pages"), c_int(q.shape[0]), c_int(rank), c_int(rot_dim),
            _stream()), "latent_store")

    def latent_gather(self, pages, ctx, block_table, dense):
        """dense[t] = the cached vector at row t's (sequence, position)."""
        _check(self._fn("latent_gather")(_ptr(pages, self.dtype, "pages"), _ptr(ctx.tok_pos, torch.int32, "tok_pos"),
                                         _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(block_table, torch.int32, "block_table"),
                                         c_int(block_table.shape[1]), _ptr(dense, self.dtype, "dense"), c_int(dense.shape[0]),
                                         c_int(dense.shape[1]), _stream()), "latent_gather")

    def latent_heads(self, q, kv, dense, rank, ctx, table, kt, vt, qt, n_heads, dim, rot_dim, v_dim, hd):
        """Keys [Wuk c | rotated part | 0], values [Wuv c | 0] and queries [q | 0] per head, `hd` wide, keys and values
        into pages of their own by `table` (a prompt step from position 0)."""
        _check(self._fn("latent_heads")(self._view(q, "q"), c_int(q.stride(0)), self._view(kv, "kv"), c_int(kv.stride(0)),
                                        self._view(dense, "dense"), c_int(dense.stride(0)), c_int(rank),
                                        _ptr(ctx.tok_pos, torch.int32, "tok_pos"), _ptr(ctx.tok_seq, torch.int32, "tok_seq"),
                                        _ptr(table, torch.int32, "table"), c_int(table.shape[1]), _ptr(kt, self.dtype, "kt"),
                                        _ptr(vt, self.dtype, "vt"), _ptr(qt, self.dtype, "qt"), c_int(q.shape[0]), c_int(n_heads),
                                        c_int(dim), c_int(rot_dim), c_int(v_dim), c_int(hd), _stream()), "latent_heads")

    def latent_absorb(self, q, wuk, qa, n_heads, dim, rot_dim, rank, scale):
        """qa float32 [T, H, rank + rot_dim] = scale * [Wuk_h^T q_h[:dim] | q_h[dim:]] for every head."""
        if q.dtype != self.dtype:
            raise KernelError(f"latent_absorb: q has dtype {q.dtype}, expected {self.dtype}")
        _check(self._fn("latent_absorb")(self._view(q, "q"), c_int(q.stride(0)), _ptr(wuk, self.dtype, "wuk"),
                                         _ptr(qa, torch.float32, "qa"), c_int(q.shape[0]), c_int(n_heads), c_int(dim),
                                         c_int(rot_dim), c_int(rank), c_float(scale), _stream()), "latent_absorb")

    def latent_attn(self, qa, pages, ctx, block_table, part, n_heads, rank, rot_dim, n_split):
        _check(self._fn("latent_attn")(
            _ptr(qa, torch.float32, "qa"), _ptr(pages, self.dtype, "pages"), _ptr(ctx.tok_pos, torch.int32, "tok_pos"),
            _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]),
            _ptr(part, torch.float32, "part"), c_int(qa.shape[0]), c_int(n_heads), c_int(rank), c_int(rot_dim), c_int(n_split),
            _stream()), "latent_attn")

    def latent_expand(self, part, olat, wuv, out, n_heads, v_dim, rank, n_split):
        """Merges the splits of `part` into olat float32 [T, H, rank] (scratch), then out[t, h] = Wuv_h olat[t, h]."""
        _check(self._fn("latent_expand")(_ptr(part, torch.float32, "part"), _ptr(olat, torch.float32, "olat"),
                                         _ptr(wuv, self.dtype, "wuv"), _ptr(out, self.dtype, "out"), c_int(out.shape[1]),
                                         c_int(out.shape[0]), c_int(n_heads), c_int(v_dim), c_int(rank), c_int(n_split), _stream()),
               "latent_expand")
        LAUNCHES[0] += 1

    def selective_scan(self, x, dt_raw, dt_bias, a_log, dskip, bc, b_col, c_col, z, state, ctx, out, inner, n_state):
        """x, z [T, I] views and bc [T, ...] of the element type (B at b_col, C at c_col), dt_raw float32 [T, I],
        dt_bias, a_log [I, N], dskip float32; state float32 [slots, I, N] (read and advanced); out [T, I]."""
        if tuple(state.shape[1:]) != (inner, n_state) or dt_raw.dtype != torch.float32:
            raise KernelError(f"selective_scan shapes: state {tuple(state.shape)}, dt {dt_raw.dtype}")
        for t, name in ((x, "x"), (z, "z"), (bc, "bc"), (out, "out")):
            if t.dtype != self.dtype:
                raise KernelError(f"selective_scan: {name} has dtype {t.dtype}, expected {self.dtype}")
        _check(self._fn("selective_scan")(
            self._view(x, "x"), c_int(x.stride(0)), _ptr(dt_raw, torch.float32, "dt_raw"), c_int(dt_raw.shape[1]),
            _ptr(dt_bias, torch.float32, "dt_bias"), _ptr(a_log, torch.float32, "a_log"), _ptr(dskip, torch.float32, "dskip"),
            c_int(1), self._view(bc, "bc"), c_int(bc.stride(0)), c_int(b_col), c_int(c_col), self._view(z, "z"),
            c_int(z.stride(0)), _ptr(state, torch.float32, "state"), _ptr(ctx.seq_start, torch.int32, "seq_start"),
            _ptr(ctx.slots, torch.int32, "slots"), self._view(out, "out"), c_int(out.stride(0)), c_int(ctx.n_seqs),
            c_int(max(1, ctx.max_new)), c_int(inner), c_int(n_state), _stream()), "selective_scan")

    ROUTERS = {"grouped_sigmoid": 0, "top_softmax": 1, "grouped_softmax": 2}

    def moe_route(self, z, correction, idx, wgt, n_groups, keep, top, scale, top_softmax=False, router=None):
        """z float32 [T, E] the router's logits -> idx int32 [T, top] the chosen experts, wgt float32 [T, top] their weights.
        `top_softmax`: the highest z + correction (a bias; may be None) are chosen and weigh with the softmax over the
        chosen ones alone; "grouped_softmax": scores are the softmax over all experts, a run of experts is rated by its best
        score, the best open experts weigh with their scores as they are (times scale); else sigmoid scores, a correction
        that only enters the picking, runs of experts rated by their best two."""
        T, E = z.shape
        mode = self.ROUTERS[router] if router is not None else (1 if top_softmax else 0)
        _check(self._fn("moe_route")(_ptr(z, torch.float32, "z"), _ptr(correction, torch.float32, "correction"), c_int(1),
                                     _ptr(idx, torch.int32, "idx"), _ptr(wgt, torch.float32, "wgt"), c_int(T), c_int(E),
                                     c_int(n_groups), c_int(keep), c_int(top), c_float(scale), c_int(mode),
                                     _stream()), "moe_route")

    def moe_pairs(self, h, wup, wdown, idx, wgt, hid, out, glu=None, tiled=False):
        """wup [E, F, K], wdown [E, N, F]; out float32 [top, T, N] partial sums over a token's chosen experts.
        `glu` = (limit, alpha): wup is [E, 2 F, K] (gate rows, then up rows; `tiled`: 8 gate rows and their 8 up rows in
        turn) and the clamped gate is the activation."""
        T, K = h.shape
        top = idx.shape[1]
        F = wdown.shape[2]
        _check(self._fn("moe_pairs")(self._view(h, "h"), c_int(h.stride(0)), _ptr(wup, self.dtype, "wup"),
                                     _ptr(wdown, self.dtype, "wdown"), _ptr(idx, torch.int32, "idx"), _ptr(wgt, torch.float32, "wgt"),
                                     _ptr(hid, self.dtype, "hid"), _ptr(out, torch.float32, "out"), c_int(T), c_int(top), c_int(K),
                                     c_int(F), c_int(wdown.shape[1]), c_int(0 if glu is None else 2 if tiled else 1),
                                     c_float(0.0 if glu is None else glu[0]), c_float(0.0 if glu is None else glu[1]), _stream()),
               "moe_pairs")

    def glu_clamp(self, gu, out, limit, alpha, rows_used=None, tiled=False):
        """out [rows, F] = the clamped gate of gu [rows, 2 F] (F gate sums, then F up sums a row; `tiled`: 8 and 8 in turn):
        g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit). `rows_used`: an int32 on the
        device, rows from there on stay."""
        _check(self._fn("glu_clamp")(_ptr(gu, self.dtype, "gu"), _ptr(out, self.dtype, "out"), c_int(out.shape[0]),
                                     c_int(out.shape[1]), c_float(limit), c_float(alpha), _ptr(rows_used, torch.int32, "rows_used"),
                                     c_int(1 if tiled else 0), _stream()), "glu_clamp")

    def moe_group_rows(self, idx, counts, offsets, pair_of_row, row_of_pair=None, tile_group=None, pad=1):
        """Groups the (token, expert) pairs of idx [T, top] by expert. counts int32 [E] must be zero and is left
        zero; offsets int32 [E + 1] the experts' first rows; pair_of_row int32 [rows] (-1: no pair); row_of_pair
        int32 [T * top] the inverse. pad > 1: every expert's rows start at a multiple of pad, and
        tile_group int32 [rows / pad] names the expert of every pad rows."""
        T, top = idx.shape
        _check(self._fn("moe_group_rows")(_ptr(idx, torch.int32, "idx"), _ptr(counts, torch.int32, "counts"),
                                          _ptr(offsets, torch.int32, "offsets"), _ptr(pair_of_row, torch.int32, "pair_of_row"),
                                          _ptr(row_of_pair, torch.int32, "row_of_pair"), _ptr(tile_group, torch.int32, "tile_group"),
                                          c_int(T), c_int(top), c_int(counts.shape[0]), c_int(pad), c_int(pair_of_row.shape[0]),
                                          _stream()), "moe_group_rows")
        LAUNCHES[0] += 4

    def moe_grouped(self, h, wup, wdown, wgt, offsets, pair_of_row, hid, out, glu=None, raw=None, tiled=False):
        """The experts' products over rows grouped without padding (`moe_group_rows` with pad 1), float32 sums on
        the FMA units; out float32 [top, T, N]. `glu` = (limit, alpha) with `raw` [T * top, 2 F] scratch: gated experts
        (`tiled` as for `moe_pairs`)."""
        T, K = h.shape
        top = wgt.shape[1]
        _check(self._fn("moe_grouped")(self._view(h, "h"), c_int(h.stride(0)), _ptr(wup, self.dtype, "wup"),
                                       _ptr(wdown, self.dtype, "wdown"), _ptr(wgt, torch.float32, "wgt"),
                                       _ptr(offsets, torch.int32, "offsets"), _ptr(pair_of_row, torch.int32, "pair_of_row"),
                                       _ptr(hid, self.dtype, "hid"), _ptr(out, torch.float32, "out"), c_int(T), c_int(top),
                                       c_int(wup.shape[0]), c_int(K), c_int(wdown.shape[2]), c_int(wdown.shape[1]),
                                       c_int(0 if glu is None else 2 if tiled else 1), c_float(0.0 if glu is None else glu[0]),
                                       c_float(0.0 if glu is None else glu[1]), _ptr(raw, self.dtype, "raw"), _stream()),
               "moe_grouped")
        LAUNCHES[0] += 1

    def moe_gather_rows(self, h, pair_of_row, top, xs):
        """xs[row] = h[pair_of_row[row] // top], zeros where a row holds no pair."""
        _check(self._fn("moe_gather_rows")(self._view(h, "h"), c_int(h.stride(0)), _ptr(pair_of_row, torch.int32, "pair_of_row"),
                                           c_int(top), _ptr(xs, self.dtype, "xs"), c_int(xs.shape[0]), c_int(xs.shape[1]), _stream()),
               "moe_gather_rows")

    def moe_combine(self, ys, row_of_pair, wgt, out):
        """out[t] = sum_k wgt[t, k] * ys[row_of_pair[t * top + k]], float32 [T, N]."""
        T, top = wgt.shape
        _check(self._fn("moe_combine")(_ptr(ys, torch.float32, "ys"), _ptr(row_of_pair, torch.int32, "row_of_pair"),
                                       _ptr(wgt, torch.float32, "wgt"), _ptr(out, torch.float32, "out"), c_int(T), c_int(top),
                                       c_int(out.shape[1]), _stream()), "moe_combine")


class GateKernels:
    """Launchers of gate_kernels.cuh. `dtype` is the element type of activations and weights; norms, gates,
    angles and the residual sum are float32 in both sets."""

    def __init__(self, dtype: torch.dtype):
        if dtype not in _SUFFIX:
            raise KernelError(f"no kernels for {dtype}; supported: float32, bfloat16")
        self.dtype, self.suffix = dtype, _SUFFIX[dtype]
        self.lib = load_library("gate_" + self.suffix)
        self._fns: dict[str, object] = {}

    _fn = SequenceKernels._fn
    _flag = SequenceKernels._flag
    _view = staticmethod(SequenceKernels._view)

    def qk_norm_store(self, c, q_out, tok_pos, tok_seq, block_table, cos_sin, kpages, vpages, n_heads, n_kv, head_dim, v_dim,
                      rot, interleaved, q_weight, k_weight, eps):
        """Row t of c (float32 or element type; a view) holds [queries | keys | values] of a token. Queries and keys are
        each divided by the root mean square of their whole part and multiplied by q_weight / k_weight (None: as
        they are), turned by the table over their first `rot` dims, and go to q_out [T, n_heads * head_dim] and, with
        the values, to the rows' places in the cache pages (n_kv == 0: queries only)."""
        w_f32 = 0
        for w in (q_weight, k_weight):
            if w is not None:
                w_f32 = self._flag(w, "norm weight")
        _check(self._fn("qk_norm_store")(
            self._view(c, "c"), c_int(self._flag(c, "c")), c_int(c.stride(0)), self._view(q_out, "q_out"), c_int(q_out.stride(0)),
            _ptr(tok_pos, torch.int32, "tok_pos"), _ptr(tok_seq, torch.int32, "tok_seq"),
            _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1] if block_table is not None else 0),
            _ptr(cos_sin, torch.float32, "cos_sin"), _ptr(kpages, self.dtype if kpages is not None else None, "kpages"),
            _ptr(vpages, self.dtype if vpages is not None else None, "vpages"), c_int(c.shape[0]), c_int(n_heads), c_int(n_kv),
            c_int(head_dim), c_int(v_dim), c_int(rot), c_int(1 if interleaved else 0), _ptr(q_weight, None, "q_weight"),
            _ptr(k_weight, None, "k_weight"), c_int(w_f32), c_float(eps), _stream()), "qk_norm_store")

    FUSED_CONV_MAX_WIDTH = 200 * 1024 // 4      # the row stays in shared memory as floats

    def conv_qk_norm_store(self, y, conv_weight, taps, state, ctx, q_out, block_table, cos_sin, kpages, vpages, n_heads, n_kv,
                           head_dim, v_dim, rot, interleaved, q_weight, k_weight, eps):
        """`qk_norm_store` behind a short causal convolution, in one kernel: y [T, C] (element type; a view) is the projection
        [queries | keys | values], conv_weight [C, taps], state float32 [slots, taps - 1, C] holds each sequence's last
        taps - 1 projected rows before the step and after it. C <= FUSED_CONV_MAX_WIDTH."""
        T, C = y.shape
        if (C != (n_heads + n_kv) * head_dim + n_kv * v_dim or tuple(conv_weight.shape) != (C, taps) or taps < 2
                or tuple(state.shape[1:]) != (taps - 1, C) or C > self.FUSED_CONV_MAX_WIDTH or y.dtype != self.dtype):
            raise KernelError(f"conv_qk_norm_store shapes: y {tuple(y.shape)} {y.dtype}, weight {tuple(conv_weight.shape)}, "
                              f"state {tuple(state.shape)}")
        w_f32 = 0
        for w in (q_weight, k_weight):
            if w is not None:
                w_f32 = self._flag(w, "norm weight")
        _check(self._fn("conv_qk_norm_store")(
            self._view(y, "y"), c_int(y.stride(0)), _ptr(conv_weight, None, "conv_weight"), c_int(self._flag(conv_weight, "conv_weight")),
            c_int(taps), _ptr(state, torch.float32, "state"), _ptr(ctx.seq_start, torch.int32, "seq_start"),
            _ptr(ctx.tok_seq, torch.int32, "tok_seq"), _ptr(ctx.slots, torch.int32, "slots"), c_int(ctx.n_seqs),
            c_int(1 if ctx.is_decode else 0), self._view(q_out, "q_out"), c_int(q_out.stride(0)),
            _ptr(ctx.tok_pos, torch.int32, "tok_pos"), _ptr(block_table, torch.int32, "block_table"),
            c_int(block_table.shape[1] if block_table is not None else 0), _ptr(cos_sin, torch.float32, "cos_sin"),
            _ptr(kpages, self.dtype if kpages is not None else None, "kpages"),
            _ptr(vpages, self.dtype if vpages is not None else None, "vpages"), c_int(T), c_int(n_heads), c_int(n_kv),
            c_int(head_dim), c_int(v_dim), c_int(rot), c_int(1 if interleaved else 0), _ptr(q_weight, None, "q_weight"),
            _ptr(k_weight, None, "k_weight"), c_int(w_f32), c_float(eps), _stream()), "conv_qk_norm_store")
        if not ctx.is_decode:
            LAUNCHES[0] += 1

    def head_gate(self, o, g, n_heads, v_dim):
        """o [T, n_heads * v_dim] (element type) *= sigmoid(g [T, n_heads]) per head; g a view, float32 or element type."""
        _check(self._fn("head_gate")(self._view(o, "o"), c_int(o.stride(0)), self._view(g, "g"), c_int(self._flag(g, "g")),
                                     c_int(g.stride(0)), c_int(o.shape[0]), c_int(n_heads), c_int(v_dim), _stream()), "head_gate")

    def add_cast(self, x, delta, xb):
        """x float32 [T, d] += delta (None, [T, d] float32 or element type, or float32 [P, T, d] partial sums);
        xb [T, d] = x in the element type."""
        P = 0 if delta is None else (delta.shape[0] if delta.dim() == 3 else 1)
        if delta is not None and (tuple(delta.shape[-2:]) != tuple(x.shape) or not delta.is_contiguous()):
            raise KernelError(f"addend {tuple(delta.shape)} does not fit the stream {tuple(x.shape)}")
        _check(self._fn("add_cast")(_ptr(x, torch.float32, "x"), _ptr(delta, None, "delta"),
                                    c_int(self._flag(delta, "delta") if delta is not None else 0), c_int(P),
                                    _ptr(xb, self.dtype, "xb"), ctypes.c_longlong(x.numel()), _stream()), "add_cast")

    def add_list_cast(self, x, addends, xb=None, vec=None):
        """x float32 [T, d] += every tensor of `addends` ([T, d] float32 or element type, or float32 [P, T, d] partial sums, added
        in their order) and `vec` (float32 [d], on every row); xb (element type [T, d], optional) = the stream rounded."""
        if len(addends) > 8:
            raise KernelError(f"{len(addends)} addends at once; the kernel takes 8")
        for a in addends:
            if tuple(a.shape[-2:]) != tuple(x.shape) or not a.is_contiguous() or not a.is_cuda or a.dim() not in (2, 3):
                raise KernelError(f"addend {tuple(a.shape)} does not fit the stream {tuple(x.shape)}")
        n = len(addends)
        ptrs = (c_void_p * max(n, 1))(*[a.data_ptr() for a in addends])
        f32 = (c_int * max(n, 1))(*[self._flag(a, "addend") for a in addends])
        parts = (c_int * max(n, 1))(*[a.shape[0] if a.dim() == 3 else 1 for a in addends])
        _check(self._fn("add_list_cast")(_ptr(x, torch.float32, "x"), ptrs, f32, parts, c_int(n), _ptr(vec, torch.float32, "vec"),
                                         c_int(x.shape[1]), _ptr(xb, self.dtype if xb is not None else None, "xb"),
                                         ctypes.c_longlong(x.numel()), _stream()), "add_list_cast")

    def gelu_mul_rows(self, a, ids, table, col0, out):
        """out [T, D] = gelu_tanh(a [T, D]) * table[ids[t], col0 : col0 + D]."""
        _check(self._fn("gelu_mul_rows")(self._view(a, "a"), c_int(a.stride(0)), _ptr(ids, torch.int32, "ids"),
                                         _ptr(table, self.dtype, "table"), c_int(table.shape[1]), c_int(col0),
                                         _ptr(out, self.dtype, "out"), c_int(a.shape[0]), c_int(a.shape[1]), _stream()),
               "gelu_mul_rows")

    def add_rms_normed(self, x, y, weight, eps, norm=None, rows=None, vec=None, dyt=None):
        """x float32 [T, d] += y / sqrt(mean(y^2) + eps) * weight; y [T, d] or [P, T, d] partial sums (float32 or element type).
        `norm` = (weight2, eps2, out): in the same pass out (element type) = x / sqrt(mean(x^2) + eps2) * weight2 of the
        stream as it then stands; with `rows` (int32 on the device) only those rows are worked on and out has a row for each.
        `dyt` = (weight2, bias2, alpha2, out), all float32: the norm that follows is tanh(alpha2 x) * weight2 + bias2 instead.
        `vec` (float32 [d]): added to every row worked on, with the addend."""
        P = y.shape[0] if y.dim() == 3 else 1
        b2, alpha2 = None, 0.0
        if dyt is not None:
            if norm is not None:
                raise KernelError("one norm follows the sum, not two")
            w2, b2, alpha2, out = dyt
            norm = (w2, 0.0, out)
            if w2.dtype != torch.float32 or b2.dtype != torch.float32 or b2.shape[0] != x.shape[1]:
                raise KernelError("the norm without statistics takes float32 weight and bias of the stream's width")
        if tuple(y.shape[-2:]) != tuple(x.shape) or not y.is_contiguous() or (rows is not None and norm is None):
            raise KernelError(f"y {tuple(y.shape)} does not fit the stream {tuple(x.shape)}")
        if vec is not None and (vec.dtype != torch.float32 or vec.numel() != x.shape[1]):
            raise KernelError(f"the row vector {tuple(vec.shape)} {vec.dtype} does not fit the stream {tuple(x.shape)}")
        w2, eps2, out = norm if norm is not None else (None, 0.0, None)
        n_out = 0 if norm is None else (x.shape[0] if rows is None else rows.shape[0])
        if norm is not None and (tuple(out.shape) != (n_out, x.shape[1]) or not out.is_contiguous() or w2.shape[0] != x.shape[1]):
            raise KernelError(f"the norm's output {tuple(out.shape)} does not fit {n_out} rows of the stream {tuple(x.shape)}")
        _check(self._fn("add_rms_normed")(_ptr(x, torch.float32, "x"), _ptr(y, None, "y"), c_int(self._flag(y, "y")), c_int(P),
                                          c_int(x.shape[0]), _ptr(weight, None, "weight"), c_int(self._flag(weight, "weight")),
                                          c_int(x.shape[1]), c_float(eps), _ptr(rows, torch.int32, "rows"), c_int(n_out),
                                          _ptr(w2, None, "weight2"), c_int(self._flag(w2, "weight2") if w2 is not None else 0),
                                          c_float(eps2), _ptr(out, self.dtype if out is not None else None, "out"),
                                          _ptr(vec, torch.float32, "vec"), _ptr(b2, torch.float32, "bias2"), c_float(alpha2), _stream()),
               "add_rms_normed")

    def softcap(self, x, cap, scale=1.0):
        """x float32 = cap * tanh(x * scale / cap), in place; without a cap (None or 0), x * scale."""
        _check(self._fn("softcap")(_ptr(x, torch.float32, "x"), ctypes.c_longlong(x.numel()), c_float(cap or 0.0), c_float(scale),
                                   _stream()), "softcap")


class CastKernels:
    """bfloat16 <-> float32 copies (a matrix stored in 32-bit inside a bfloat16 model)."""

    def __init__(self):
        self.lib = load_library("bf16")

    def to_f32(self, src, dst):
        fn = self.lib.sllm_cast_bf16_to_f32
        fn.restype = c_int
        _check(fn(_ptr(src, torch.bfloat16, "src"), _ptr(dst, torch.float32, "dst"), c_longlong(src.numel()), _stream()),
               "cast_bf16_to_f32")

    def to_bf16(self, src, dst):
        fn = self.lib.sllm_cast_f32_to_bf16
        fn.restype = c_int
        _check(fn(_ptr(src, torch.float32, "src"), _ptr(dst, torch.bfloat16, "dst"), c_longlong(src.numel()), _stream()),
               "cast_f32_to_bf16")


class RandomKernels:
    """Fills tensors with the counter-based generator of random-weights mode (lib_random.cu)."""

    def __init__(self):
        self.lib = load_library("random")
        self.lib.sllm_fill_normal.restype = c_int
        self.lib.sllm_fill_integer.restype = c_int

    def fill_normal(self, out, seed: int, index: int, mean: float, std: float):
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"fill_normal writes float32 or bfloat16, not {out.dtype}")
        _check(self.lib.sllm_fill_normal(_ptr(out, None, "out"), c_int(0 if out.dtype == torch.float32 else 1),
                                         c_longlong(out.numel()), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                                         ctypes.c_uint(index), ctypes.c_double(mean), ctypes.c_double(std), _stream()),
               "fill_normal")

    def fill_integer(self, out, seed: int, index: int, modulus: int):
        _check(self.lib.sllm_fill_integer(_ptr(out, torch.int32, "out"), c_longlong(out.numel()),
                                          ctypes.c_ulonglong(seed & (2 ** 64 - 1)), ctypes.c_uint(index),
                                          ctypes.c_uint(modulus), _stream()), "fill_integer")


class ProbeKernels:
    """Measuring sticks for benchmarks (lib_probe.cu)."""

    def __init__(self):
        self.lib = load_library("probe")
        self.lib.sllm_fma_loop.restype = c_int

    def fma_tflops(self, device="cuda:0", blocks_per_sm: int = 8, iters: int = 1 << 15, repeats: int = 5) -> float:
        """Best-of-`repeats` rate of float fused multiply-adds (2 operations each) in TFLOP/s."""
        dev = torch.device(device)
        blocks = torch.cuda.get_device_properties(dev).multi_processor_count * blocks_per_sm
        out = torch.empty(blocks * 256, dtype=torch.float32, device=dev)
        best = 0.0
        for i in range(repeats + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _check(self.lib.sllm_fma_loop(_ptr(out, torch.float32, "out"), c_int(blocks), c_int(iters), _stream()), "fma_loop")
            e1.record()
            e1.synchronize()
            if i:
                best = max(best, blocks * 256 * iters * 16 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        return best


class SamplingKernels:
    STRATEGIES = {"greedy": 0, "temperature": 1, "top_k": 2, "top_p": 3}
    PARAM_WORDS = 8   # int32 words per row: strategy, temperature, top_k, top_p, seed lo/hi, draw lo/hi

    def __init__(self):
        self.lib = load_library("sampling")

    def sample_rows(self, logits, params, out):
        """logits float32 [n, V] (row stride = logits.stride(0)); params int32 [n, 8]; out int32 [n]."""
        if logits.dim() != 2 or logits.stride(1) != 1:
            raise KernelError("logits must be [rows, vocab] with unit column stride")
        n, V = logits.shape
        fn = self.lib.sllm_sample_rows
        fn.restype = c_int
        if not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("logits must be float32 on a CUDA device")
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V),
                  _ptr(params, torch.int32, "params"), _ptr(out, torch.int32, "out"), _stream()), "sample_rows")

    STATE_WORDS = 8   # int32 words of a sequence's state record: pos, generated, last token, flags, key x2, counter x2

    def sample_rows_state(self, logits, options, state, slots, pos_after, stop_ids, out):
        """The same, every row's sampling key and draw counter read from (and advanced in) its
        sequence's record state[slots[row]]; options int32 [4] on the device; stop_ids int32 [n] or None."""
        if logits.dim() != 2 or logits.stride(1) != 1 or not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("logits must be float32 [rows, vocab] with unit column stride on a CUDA device")
        n, V = logits.shape
        if state.dim() != 2 or state.shape[1] != self.STATE_WORDS or slots.shape[0] < n or out.shape[0] < n:
            raise KernelError("sample_rows_state: state must be [slots, 8] and slots/out must cover every row")
        fn = self.lib.sllm_sample_rows_state
        fn.restype = c_int
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V), _ptr(options, torch.int32, "options"),
                  _ptr(state, torch.int32, "state"), _ptr(slots, torch.int32, "slots"), _ptr(pos_after, torch.int32, "pos_after"),
                  _ptr(stop_ids, torch.int32, "stop_ids"), c_int(0 if stop_ids is None else stop_ids.numel()),
                  _ptr(out, torch.int32, "out"), _stream()), "sample_rows_state")

    def repeat_penalty(self, logits, recent, counts, penalty, last_n):
        n, V = logits.shape
        fn = self.lib.sllm_repeat_penalty
        fn.restype = c_int
        _check(fn(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), c_int(n), c_int(V),
                  _ptr(recent, torch.int32, "recent"), c_int(recent.shape[1]), _ptr(counts, torch.int32, "counts"),
                  _ptr(penalty, torch.float32, "penalty"), c_int(last_n), _stream()), "repeat_penalty")
