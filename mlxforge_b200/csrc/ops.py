"""Python-side launchers of the CUDA kernels, taking torch tensors.

These are thin: they check what the kernel cannot check for itself, pass raw
pointers and the current stream, and raise ``KernelError`` on a refusal.
"""
from __future__ import annotations

from ctypes import c_void_p
from typing import Optional

import torch

from .binding import KernelError, check, count_launches, library

F32, BF16 = 0, 1


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensor dtype {t.dtype} is neither float32 nor bfloat16")


# The current stream's handle without building a torch.cuda.Stream object for it (that costs
# about 15 us a call, and every kernel launch asks): torch's own binding for it, where present.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel operands must be contiguous CUDA tensors "
                              f"(got device={t.device}, contiguous={t.is_contiguous()})")


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[tokens[t]] * scale, into the 32-bit residual stream."""
    _need_cuda(table, tokens, out)
    T, H = out.shape
    check(library().mf_embed(table.data_ptr(), dtype_code(table), tokens.data_ptr(), out.data_ptr(), T, H, scale,
                             _stream()), "embed")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    _need_cuda(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    n = out.shape[0]
    check(library().mf_add_rmsnorm(resid.data_ptr(), _ptr(delta), dtype_code(delta) if delta is not None else F32,
                                   weight.data_ptr(), eps, out.data_ptr(), dtype_code(out), _ptr(rows), n, H,
                                   _stream()), "add_rmsnorm")


def residual_add(resid: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(resid, delta)
    check(library().mf_residual_add(resid.data_ptr(), delta.data_ptr(), dtype_code(delta), resid.numel(),
                                    _stream()), "residual_add")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, freqs: Optional[torch.Tensor], q_out: torch.Tensor,
                  k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                  rotary_dim: int, write_kv: bool, precise: bool) -> None:
    _need_cuda(qkv, positions, seq_of_token, block_table, freqs, q_out, k_pool, v_pool)
    T = qkv.shape[0]
    check(library().mf_rope_kv_write(qkv.data_ptr(), dtype_code(qkv), T, n_heads, n_kv, head_dim, rotary_dim,
                                     positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                     block_table.shape[1], page_size, _ptr(freqs), q_out.data_ptr(),
                                     k_pool.data_ptr(), v_pool.data_ptr(), int(write_kv), int(precise),
                                     _stream()), "rope_kv_write")


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}
STREAM_UNARY = 16      # mode of the few-row product with an activation without a gate: STREAM_UNARY + code


def activation_code(act: str) -> int:
    try:
        return ACTIVATIONS[act]
    except KeyError:
        raise KernelError(f"unknown gate activation '{act}' (one of {sorted(ACTIVATIONS)})") from None


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int, act: str = "silu") -> None:
    """out = act(gate) * up for gate and up interleaved in groups of ``group`` columns."""
    _need_cuda(gu, out)
    T, I = out.shape
    check(library().mf_gated_act(gu.data_ptr(), out.data_ptr(), dtype_code(gu), T, I, group, activation_code(act),
                                 _stream()), "gated_act")


def unary_act(x: torch.Tensor, out: torch.Tensor, act: str) -> None:
    """out = act(x), element by element in 32-bit (``out`` may be ``x``)."""
    _need_cuda(x, out)
    if x.dtype != out.dtype or x.numel() != out.numel():
        raise KernelError("unary_act: input and output of one dtype and size")
    check(library().mf_unary_act(x.data_ptr(), out.data_ptr(), dtype_code(x), x.numel(), activation_code(act),
                                 _stream()), "unary_act")


def add_rmsnorm_pair(resid: torch.Tensor, d1: Optional[torch.Tensor], d2: Optional[torch.Tensor], w1: torch.Tensor,
                     w2: Optional[torch.Tensor], eps: float, out1: torch.Tensor, out2: Optional[torch.Tensor],
                     rows: Optional[torch.Tensor] = None) -> None:
    """``resid += d1 + d2`` (either may be None), then ``out1 = rmsnorm(resid) * w1`` and, where asked for,
    ``out2 = rmsnorm(resid) * w2``.  With ``rows`` only those rows are produced and ``resid`` stays."""
    _need_cuda(resid, d1, d2, w1, w2, out1, out2, rows)
    if d1 is not None and d2 is not None and d1.dtype != d2.dtype:
        raise KernelError("add_rmsnorm_pair: the two deltas must have one dtype")
    d = d1 if d1 is not None else d2
    check(library().mf_add_rmsnorm_pair(resid.data_ptr(), _ptr(d1), _ptr(d2), dtype_code(d) if d is not None else F32,
                                        w1.data_ptr(), _ptr(w2), eps, out1.data_ptr(), _ptr(out2), dtype_code(out1),
                                        _ptr(rows), out1.shape[0], resid.shape[-1], _stream()), "add_rmsnorm_pair")


def rope_store(qk: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
               page_size: int, inv_f: Optional[torch.Tensor], inv_d: Optional[torch.Tensor], q_out: torch.Tensor,
               k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rotary_dim: int,
               pairs: bool, write_kv: bool, v_from_k: bool, ld: Optional[int] = None) -> None:
    """Rotation of queries and keys (``pairs``: channel 2i with 2i+1, else i with i + rotary_dim/2) with the
    cache write; ``v_from_k``: the rows hold no values and the value pages get the keys before rotation.
    ``inv_d`` (float64 inverse wavelengths) selects angles in double, else ``inv_f`` (float32).  Rows of
    ``qk`` are ``ld`` elements apart (default: as wide as their heads)."""
    _need_cuda(positions, seq_of_token, block_table, inv_f, inv_d, q_out, k_pool, v_pool)
    if ld is None:
        ld = (n_heads + (1 if v_from_k else 2) * n_kv) * head_dim
    check(library().mf_rope_store(qk.data_ptr(), ld, dtype_code(qk), qk.shape[0], n_heads, n_kv, head_dim, rotary_dim,
                                  1 if pairs else 0, positions.data_ptr(), seq_of_token.data_ptr(),
                                  block_table.data_ptr(), block_table.shape[1], page_size, _ptr(inv_f), _ptr(inv_d),
                                  q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), int(write_kv), int(v_from_k),
                                  _stream()), "rope_store")


def attention_generic_ex(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                         positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                         page_size: int, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                         v_dim: int, v_ld: int, keep_first: int = 0, sink: Optional[torch.Tensor] = None,
                         gate: Optional[torch.Tensor] = None, gate_ld: int = 0, softcap: float = 0.0) -> None:
    """The block-per-token attention with its options: values ``v_dim`` wide in rows ``v_ld`` apart
    (``v_pool`` may be ``k_pool``), the first ``keep_first`` keys kept beside the window, a sink per head in
    the softmax denominator, the output times sigmoid(``gate``) (rows ``gate_ld`` apart)."""
    _need_cuda(q, k_pool, v_pool, out, positions, seq_of_token, block_table, sink)
    check(library().mf_attention_generic_ex(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                            dtype_code(q), q.shape[0], n_heads, n_kv, head_dim, positions.data_ptr(),
                                            seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                            page_size, scale, window, v_dim, v_ld, keep_first, _ptr(sink),
                                            _ptr(gate), gate_ld, float(softcap or 0.0), _stream()), "attention_generic")


def attention_tc_ok(head_dim: int, v_dim: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels with options take these sizes."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256 and v_dim % 16 == 0 and 0 < v_dim <= head_dim \
        and page_size % 16 == 0


def attention_prefill_ex(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                         seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_ctx_len: torch.Tensor,
                         table_row0: int, max_q_len: int, block_table: torch.Tensor, page_size: int, n_heads: int,
                         n_kv: int, head_dim: int, scale: float, window: int, v_dim: int, v_in_k: bool,
                         keep_first: int = 0, sink: Optional[torch.Tensor] = None,
                         gate: Optional[torch.Tensor] = None, gate_ld: int = 0, softcap: float = 0.0) -> None:
    """``attention_prefill`` with options: values ``v_dim`` wide (``v_in_k``: the first channels of the keys),
    kept first keys, a sink per head, the output times sigmoid(``gate``).  bfloat16, the mma.sync kernel."""
    _need_cuda(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, block_table, sink)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_ex: bfloat16 only")
    check(library().mf_attention_prefill_ex(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                            seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_ctx_len.data_ptr(),
                                            table_row0, seq_q_len.shape[0], max_q_len, n_heads, n_kv, head_dim,
                                            block_table.data_ptr(), block_table.shape[1], page_size, scale, window,
                                            v_dim, int(v_in_k), keep_first, _ptr(sink), _ptr(gate), gate_ld,
                                            float(softcap or 0.0), _stream()), "attention_prefill_ex")


def attention_decode_ex(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                        part_o: torch.Tensor, part_ml: torch.Tensor, positions: torch.Tensor,
                        seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, n_heads: int,
                        n_kv: int, head_dim: int, scale: float, window: int, max_ctx: int, v_dim: int, v_in_k: bool,
                        keep_first: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                        gate_ld: int = 0, softcap: float = 0.0) -> None:
    """``attention_decode`` with the same options; scratch as ``attention_decode_scratch`` says for this window."""
    _need_cuda(q, k_pool, v_pool, out, part_o, part_ml, positions, seq_of_token, block_table, sink)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_decode_ex: bfloat16 only")
    n = q.shape[0]
    need_o, need_ml = attention_decode_scratch(n, n_heads, head_dim, max_ctx, window)
    if part_o.numel() < need_o or part_ml.numel() < need_ml or part_o.dtype != torch.float32:
        raise KernelError("attention_decode_ex: scratch too small")
    check(library().mf_attention_decode_ex(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                           part_o.data_ptr(), part_ml.data_ptr(), n, n_heads, n_kv, head_dim,
                                           positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                           block_table.shape[1], page_size, scale, window, max_ctx, v_dim,
                                           int(v_in_k), keep_first, _ptr(sink), _ptr(gate), gate_ld,
                                           float(softcap or 0.0), _stream()),
          "attention_decode_ex", launches=2)


def latent_prepare(proj: torch.Tensor, q_rank: int, kv_off: int, rank: int, rot: int, wq: Optional[torch.Tensor],
                   wkv: Optional[torch.Tensor], eps: float, positions: torch.Tensor, seq_of_token: torch.Tensor,
                   block_table: torch.Tensor, page_size: int, inv_f, inv_d, cq_out: Optional[torch.Tensor],
                   k_pool: torch.Tensor, write_kv: bool, pairs: bool = False, rot_dims: Optional[int] = None,
                   magnitude: float = 1.0) -> None:
    """From rows of projections [query latent | key/value latent, shared key part | ...]: the normed query
    latent into ``cq_out`` (``q_rank`` 0: there is none) and, if ``write_kv``, the normed latent and the rotated
    key part into the cache.  ``pairs``: channel 2i turns with 2i+1, else i with i + rot_dims/2; ``rot_dims`` of
    the ``rot`` channels turn (default all); cosine and sine are multiplied by ``magnitude``."""
    _need_cuda(proj, wq, wkv, cq_out, k_pool)
    launches = 0 if (q_rank == 0 and not write_kv) else 1
    check(library().mf_latent_prepare(proj.data_ptr(), dtype_code(proj), proj.shape[0], proj.shape[1], q_rank, kv_off,
                                      rank, rot, _ptr(wq), _ptr(wkv), eps, positions.data_ptr(),
                                      seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
                                      _ptr(inv_f), _ptr(inv_d), _ptr(cq_out), k_pool.data_ptr(), int(write_kv),
                                      1 if pairs else 0, rot if rot_dims is None else rot_dims, magnitude,
                                      _stream()), "latent_prepare", launches=launches)


def latent_query(q: torch.Tensor, n_heads: int, dim: int, rot: int, rank: int, positions: torch.Tensor, inv_f, inv_d,
                 q_full: torch.Tensor, q_ld: Optional[int] = None, pairs: bool = False,
                 rot_dims: Optional[int] = None, magnitude: float = 1.0) -> None:
    """The rotated part of every head's query, rotated, into columns [rank, rank + rot) of ``q_full``; rows of
    ``q`` are ``q_ld`` elements apart (default: as wide as their heads).  The rotation's options as in
    ``latent_prepare``."""
    _need_cuda(q_full)
    if q_ld is None:
        q_ld = n_heads * (dim + rot)
    check(library().mf_latent_query(q.data_ptr(), q_ld, dtype_code(q), q.shape[0], n_heads, dim, rot, rank,
                                    positions.data_ptr(), _ptr(inv_f), _ptr(inv_d), q_full.data_ptr(),
                                    1 if pairs else 0, rot if rot_dims is None else rot_dims, magnitude, _stream()),
          "latent_query", launches=1 if rot else 0)


def _gate_strides(N: int, gate_per_head: bool):
    return (1, 0) if gate_per_head else (N, 1)


def head_linear(x: torch.Tensor, x_ld: int, x_hs: int, w: torch.Tensor, out: torch.Tensor, out_ld: int, out_hs: int,
                T: int, gate: Optional[torch.Tensor] = None, gate_ld: int = 0, gate_per_head: bool = False) -> None:
    """``out[t, h, :N] = w[h] @ x[t, h, :K]`` for ``w`` [heads, N, K]; rows of ``x`` / ``out`` are ``x_ld`` /
    ``out_ld`` elements apart and heads ``x_hs`` / ``out_hs``; optionally times sigmoid(``gate[t, h * N + n]``),
    or, with ``gate_per_head``, sigmoid(``gate[t, h]``)."""
    _need_cuda(w)
    if x.dtype != w.dtype or out.dtype != w.dtype:
        raise KernelError("head_linear: operands of one dtype")
    H, N, K = w.shape
    ghs, gns = _gate_strides(N, gate_per_head)
    check(library().mf_head_linear(x.data_ptr(), x_ld, x_hs, w.data_ptr(), out.data_ptr(), out_ld, out_hs,
                                   dtype_code(w), T, H, N, K, _ptr(gate), gate_ld, ghs, gns, _stream()), "head_linear")


def head_linear_mma_ok(x: torch.Tensor, x_ld: int, x_hs: int, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel of ``head_linear`` takes these operands."""
    return (w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library().mf_head_linear_mma_ok(x_ld, x_hs, w.shape[2])))


def head_linear_mma(x: torch.Tensor, x_ld: int, x_hs: int, w: torch.Tensor, out: torch.Tensor, out_ld: int, out_hs: int,
                    T: int, gate: Optional[torch.Tensor] = None, gate_ld: int = 0, gate_per_head: bool = False) -> None:
    """``head_linear`` for many bfloat16 tokens, on the tensor cores (mma.sync tiles of 64 tokens x 64 outputs)."""
    _need_cuda(w)
    H, N, K = w.shape
    ghs, gns = _gate_strides(N, gate_per_head)
    check(library().mf_head_linear_mma(x.data_ptr(), x_ld, x_hs, w.data_ptr(), out.data_ptr(), out_ld, out_hs, T, H, N,
                                       K, _ptr(gate), gate_ld, ghs, gns, _stream()), "head_linear_mma")


def retention_prepare(proj: torch.Tensor, n_heads: int, dim: int, rot: int, k_scale: float, positions: torch.Tensor,
                      inv_f, inv_d, qk: torch.Tensor, silu: bool = False, v_out: Optional[torch.Tensor] = None,
                      v_off: int = 0) -> None:
    """Rows [queries | keys | ...] -> 32-bit [T, 2 heads dim]: both rotated, keys times ``k_scale``.  ``silu``:
    every channel passes SiLU first.  ``v_out`` [T, nv] (32-bit): the columns from ``v_off`` on, through the same
    activation."""
    _need_cuda(proj, qk, v_out)
    check(library().mf_retention_prepare(proj.data_ptr(), dtype_code(proj), proj.shape[0], proj.shape[1], n_heads, dim,
                                         rot, k_scale, positions.data_ptr(), _ptr(inv_f), _ptr(inv_d), qk.data_ptr(),
                                         int(silu), _ptr(v_out), v_off, v_out.shape[1] if v_out is not None else 0,
                                         _stream()), "retention_prepare")


def set_retention_rows(rows: int) -> None:
    """Rows of the state per block of the staged recurrence kernel (16, 32 or 64; for tests and measurements).
    Results do not depend on it beyond the order in which the row groups' partial read-outs are added."""
    check(library().mf_set_retention_rows(rows), "set_retention_rows", launches=0)


def retention_parts(dim: int, vdim: int, v: torch.Tensor, v_ld: int) -> int:
    """How many partial read-outs ``retention_recurrence`` writes for these sizes (it spreads a head's state over
    that many groups of rows where the sizes come in whole pieces); ``retention_output`` sums them."""
    return int(library().mf_retention_parts(dim, vdim, dtype_code(v), v_ld))


def retention_recurrence(qk: torch.Tensor, v: torch.Tensor, v_ld: int, decay: torch.Tensor, state: torch.Tensor,
                         batch, o_out: torch.Tensor, n_heads: int, dim: int, vdim: int) -> None:
    """``v`` points at the first value of the first token (rows ``v_ld`` elements apart).  ``o_out``
    [``retention_parts``, T, n_heads * vdim] receives the partial read-outs."""
    _need_cuda(qk, decay, state, o_out)
    if o_out.dim() != 3 or o_out.shape[0] != retention_parts(dim, vdim, v, v_ld):
        raise KernelError("retention_recurrence: o_out must hold retention_parts(...) partial read-outs")
    check(library().mf_retention_recurrence(qk.data_ptr(), v.data_ptr(), dtype_code(v), v_ld, decay.data_ptr(),
                                            state.data_ptr(), state.stride(0), batch.seq_q_start.data_ptr(),
                                            batch.seq_q_len.data_ptr(), batch.slots.data_ptr(), o_out.data_ptr(),
                                            o_out.stride(0), batch.n_seqs, n_heads, dim, vdim, _stream()),
          "retention_recurrence")


def retention_output(o: torch.Tensor, gate: torch.Tensor, gate_ld: int, eps: float, out: torch.Tensor, n_heads: int,
                     vdim: int, weight: Optional[torch.Tensor] = None, whole: bool = False,
                     gate_act: str = "silu") -> None:
    """``o`` [parts, T, n_heads * vdim]: the partial read-outs, summed here.  ``gate`` points at the first gate of
    the first token; rows are ``gate_ld`` elements apart."""
    _need_cuda(o, out)
    check(library().mf_retention_output(o.data_ptr(), o.shape[0], o.stride(0), gate.data_ptr(), dtype_code(out), gate_ld,
                                        eps, out.data_ptr(), o.shape[1], n_heads, vdim, _ptr(weight), int(whole),
                                        {"silu": 0, "sigmoid": 1}[gate_act], _stream()), "retention_output")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    check(library().mf_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(accumulate),
                                _stream()), "gemm_f32")


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                      page_size: int, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> None:
    _need_cuda(q, k_pool, v_pool, out, positions, seq_of_token, block_table)
    T = q.shape[0]
    check(library().mf_attention_generic(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                         dtype_code(q), T, n_heads, n_kv, head_dim, positions.data_ptr(),
                                         seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                         page_size, scale, window, _stream()), "attention_generic")


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                      seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_ctx_len: torch.Tensor,
                      table_row0: int, max_q_len: int, block_table: torch.Tensor, page_size: int, n_heads: int,
                      n_kv: int, head_dim: int, scale: float, window: int) -> None:
    """Attention of prompt portions, bfloat16.  ``q`` / ``out`` are the whole step's
    [T, n_heads*head_dim]; the three per-sequence arrays describe the sequences
    that start at row ``table_row0`` of ``block_table``."""
    _need_cuda(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, block_table)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    check(library().mf_attention_prefill(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                         seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_ctx_len.data_ptr(),
                                         table_row0, seq_q_len.shape[0], max_q_len, q.shape[0], n_heads, n_kv,
                                         head_dim, block_table.data_ptr(), block_table.shape[1], page_size, scale,
                                         window, kernel_status(q.device).data_ptr(), _stream()), "attention_prefill")


def set_prefill_tcgen05(on: bool) -> None:
    """Whether portions of at least 128 tokens with head size 64 take the tcgen05 attention
    kernel (the default) or every shape the mma.sync one."""
    check(library().mf_set_prefill_tcgen05(1 if on else 0), "set_prefill_tcgen05", launches=0)


def few_rows_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the few-row product kernels take these operands (rows are read in 16-byte pieces)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_STATUS = {}
_TMA_STATUS_SET = False


def kernel_status(device=None) -> torch.Tensor:
    """The device word in which kernels with bounded waits record that a wait ran out."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _STATUS[key] = t
    return t


def kernel_gave_up(code: int, device=None) -> KernelError:
    """What to do when the status word read ``code`` != 0: a kernel with bounded waits gave up,
    so what it wrote is not to be trusted.  Clears the word and everything such a kernel may
    have left half done (the decode-attention tickets), and returns the error to raise."""
    kernel_status(device).zero_()
    check(library().mf_reset_decode_tickets(_stream()), "reset_decode_tickets", launches=0)
    check(library().mf_reset_mid_rows_tickets(_stream()), "reset_mid_rows_tickets", launches=0)
    return KernelError(f"a kernel's bounded wait ran out (code {code}: 1 = copy producer, 2 = consumer); "
                       "the results of the step are invalid")


def check_kernel_status() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (reads the word back, which
    waits for the device: call it where the host waits anyway)."""
    for key, t in _STATUS.items():
        code = int(t.item())
        if code:
            raise kernel_gave_up(code, torch.device("cuda", key))


def stream_linear_has_act() -> bool:
    """Whether the few-row product has the activations without a gate in its epilogue."""
    return True


def gemm_has_act() -> bool:
    """Whether the tcgen05 product has the activations without a gate in its epilogue."""
    return True


def stream_max_rows() -> int:
    return int(library().mf_stream_max_rows())


def set_stream_tensor_copies(on: bool) -> None:
    """Whether ``stream_linear`` brings a stage with one tensor copy (widths that are a multiple
    of 64; the default) or always with one copy per row segment."""
    check(library().mf_set_stream_tensor_copies(1 if on else 0), "set_stream_tensor_copies", launches=0)


def stream_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False,
                  act: str = "silu", unary: bool = False) -> None:
    """out = x @ w^T for at most ``stream_max_rows()`` rows of bfloat16 x (out bfloat16 or
    float32), the weights streamed by bulk copies (see gemv_stream.cu); with ``swiglu`` the rows
    of w interleave gate and up in groups of 8 and out [M, N/2] is act(gate) * up; with ``unary``
    out [M, N] is act(x @ w^T), the activation applied to the 32-bit sums.
    The kernel starts fetching ``w`` before it waits for the kernel launched before it, so
    ``w`` must not be the output of that kernel (the engine's weights are written once, at
    load time)."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"stream_linear: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if swiglu and unary:
        raise KernelError("stream_linear: an activation with a gate or without one, not both")
    mode = 1 + activation_code(act) if swiglu else (STREAM_UNARY + activation_code(act) if unary else 0)
    check(library().mf_stream_linear(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out), M, N, K,
                                     mode, kernel_status(x.device).data_ptr(), _stream()),
          "stream_linear")


def mid_rows_range():
    """(fewest, most) rows of x that ``mid_linear`` takes."""
    return int(library().mf_mid_rows_min()), int(library().mf_mid_rows_max())


def mid_rows_scratch(rows: int) -> int:
    """float32 elements of scratch that ``mid_linear`` needs for ``rows`` rows of x."""
    return int(library().mf_mid_rows_scratch(rows))


def mid_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, swiglu: bool = False) -> None:
    """out = x @ w^T for 17 to 128 rows of bfloat16 x on the tcgen05 tensor cores with the weights
    streamed once (see gemm_mid_rows.cu); out bfloat16 or float32; with ``swiglu`` the rows of w
    interleave gate and up in groups of 8 and out is [M, N/2] = silu(gate) * up.  ``scratch``:
    float32, at least ``mid_rows_scratch(M)`` elements.  As with ``stream_linear``, ``w`` must not
    be the output of the kernel launched just before."""
    _need_cuda(x, w, out, scratch)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"mid_linear: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if scratch.dtype != torch.float32 or scratch.numel() < mid_rows_scratch(M):
        raise KernelError("mid_linear: scratch too small")
    check(library().mf_mid_rows_linear(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out), scratch.data_ptr(),
                                       M, N, K, 1 if swiglu else 0, kernel_status(x.device).data_ptr(), _stream()),
          "mid_linear")


def gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands (TMA needs 16-byte row strides)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False, act: str = "silu",
              unary: bool = False) -> None:
    """out = x @ w^T on the tcgen05 tensor cores (bfloat16 operands; out bfloat16 or float32);
    with ``swiglu`` the rows of w interleave gate and up in groups of 8 and out is
    [M, N/2] = act(gate) * up; with ``unary`` out [M, N] (bfloat16) is act(x @ w^T), the activation
    applied to the 32-bit sums."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    want = (M, N // 2) if swiglu else (M, N)
    if w.shape[1] != K or tuple(out.shape) != want:
        raise KernelError(f"gemm_bf16: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if (swiglu or unary) and out.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16: an epilogue with an activation writes bfloat16")
    if swiglu and unary:
        raise KernelError("gemm_bf16: an activation with a gate or without one, not both")
    if swiglu and act == "relu2":
        raise KernelError("gemm_bf16: the gated epilogue has SiLU and the tanh form of GELU")
    epi = (2 + activation_code(act) if swiglu else 4 + activation_code(act) if unary
           else (1 if out.dtype == torch.float32 else 0))
    check(library().mf_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, epi,
                                 kernel_status(x.device).data_ptr(), _stream()), "gemm_bf16")


def set_decode_tma(on: bool) -> bool:
    """Switch the TMA decode-attention kernel (head size 64) on or off; returns the previous
    setting.  Both kernels write the same partial results."""
    return bool(library().mf_set_decode_tma(1 if on else 0, kernel_status().data_ptr()))


def set_decode_merge_inside(on: bool) -> bool:
    """Whether the TMA decode-attention kernel merges its splits itself (the block that finishes a
    group's last split does it) or a merge kernel follows it; returns the previous setting."""
    return bool(library().mf_set_decode_merge_inside(1 if on else 0))


def attention_decode_split(head_dim: int) -> int:
    """Keys per split of the decode kernel for a head size."""
    return int(library().mf_attention_decode_split(head_dim))


def attention_decode_scratch(n_tokens: int, n_heads: int, head_dim: int, max_ctx: int, window: Optional[int] = None):
    """Element counts of the two float32 scratch buffers the decode kernel needs; with ``window`` (0: none)
    those of the launch with options, whose split depends on the window."""
    split = attention_decode_split(head_dim) if window is None else attention_decode_ex_split(head_dim, window)
    splits = (max_ctx + split - 1) // split
    return n_tokens * n_heads * splits * head_dim, n_tokens * n_heads * splits * 2


def attention_decode_ex_split(head_dim: int, window: int) -> int:
    """Keys per split of ``attention_decode_ex`` for a lane with this window (0: none)."""
    return int(library().mf_attention_decode_ex_split(head_dim, window))


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                     part_o: torch.Tensor, part_ml: torch.Tensor, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, n_heads: int,
                     n_kv: int, head_dim: int, scale: float, window: int, max_ctx: int,
                     unequal_contexts: bool = False) -> None:
    """Attention of tokens that are each the newest of their sequence (one query per
    sequence), bfloat16, split over the keys; ``part_o`` / ``part_ml`` are float32
    scratch of at least ``attention_decode_scratch`` elements.  ``unequal_contexts``: the
    caller knows that the contexts differ widely in length (see mf_attention_decode_hinted)."""
    _need_cuda(q, k_pool, v_pool, out, part_o, part_ml, positions, seq_of_token, block_table)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    n = q.shape[0]
    global _TMA_STATUS_SET
    if not _TMA_STATUS_SET:
        library().mf_set_decode_status(kernel_status(q.device).data_ptr())
        _TMA_STATUS_SET = True
    need_o, need_ml = attention_decode_scratch(n, n_heads, head_dim, max_ctx)
    if part_o.numel() < need_o or part_ml.numel() < need_ml or part_o.dtype != torch.float32:
        raise KernelError("attention_decode: scratch too small")
    check(library().mf_attention_decode_hinted(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                               part_o.data_ptr(), part_ml.data_ptr(), n, n_heads, n_kv, head_dim,
                                               positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                               block_table.shape[1], page_size, scale, window, max_ctx,
                                               1 if unequal_contexts else 0, _stream()),
          "attention_decode", launches=0)
    # one kernel when the TMA kernel merged its splits itself, two when a merge kernel followed
    count_launches(int(library().mf_attention_decode_launches()))


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Row r: argmax if temperature is None or temperature[r] <= 0, else an
    inverse-CDF draw from softmax(logits[r] / temperature[r]) with u[r]."""
    _need_cuda(temperature, u, out)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 CUDA rows")
    n, V = logits.shape
    split = temperature is None and V >= 16384 and n <= 4096       # greedy over a large vocabulary: two kernels
    check(library().mf_sample(logits.data_ptr(), n, V, logits.stride(0), _ptr(temperature), _ptr(u),
                              out.data_ptr(), _stream()), "sample", launches=2 if split else 1)


def apply_penalties(logits: torch.Tensor, params, histories) -> None:
    """Repetition / frequency / presence penalties, in place, over each row's
    history.  The unique ids and their counts are made on the host (the history
    lives there) and sent in one copy."""
    import numpy as np
    n = logits.shape[0]
    ids, counts, off = [], [], [0]
    for r in range(n):
        h = np.asarray(histories[r] if params[r].has_penalties else (), dtype=np.int64)
        added = 0
        if h.size:
            u, c = np.unique(h, return_counts=True)
            ids.append(u.astype(np.int32))
            counts.append(c.astype(np.int32))
            added = u.size
        off.append(off[-1] + added)
    if off[-1] == 0:
        return
    ints = np.concatenate(ids + counts + [np.asarray(off, dtype=np.int32)])
    floats = np.asarray([[p.repetition_penalty for p in params], [p.frequency_penalty for p in params],
                         [p.presence_penalty for p in params]], dtype=np.float32)
    di = torch.from_numpy(ints).to(logits.device)
    df = torch.from_numpy(floats).to(logits.device)
    m = off[-1]
    check(library().mf_apply_penalties(logits.data_ptr(), n, logits.stride(0), di[:m].data_ptr(),
                                       di[m:2 * m].data_ptr(), di[2 * m:].data_ptr(), df[0].data_ptr(),
                                       df[1].data_ptr(), df[2].data_ptr(), _stream()), "apply_penalties")


def filter_logits(logits: torch.Tensor, params) -> None:
    """top-k, top-p and min-p of every non-greedy row, in place (removed entries -inf)."""
    import numpy as np
    n, V = logits.shape
    floats = np.asarray([[0.0 if p.greedy else p.temperature for p in params], [p.top_p for p in params],
                         [p.min_p for p in params]], dtype=np.float32)
    ks = np.asarray([p.top_k for p in params], dtype=np.int32)
    df = torch.from_numpy(floats).to(logits.device)
    dk = torch.from_numpy(ks).to(logits.device)
    check(library().mf_filter_logits(logits.data_ptr(), n, V, logits.stride(0), df[0].data_ptr(), dk.data_ptr(),
                                     df[1].data_ptr(), df[2].data_ptr(), _stream()), "filter_logits")


def set_dependent_launch(on: bool) -> bool:
    """Switch programmatic dependent launch of the decode-path kernels on or off;
    returns the previous setting.  Results do not depend on it."""
    return bool(library().mf_set_pdl(1 if on else 0))


# ---------------------------------------------------------------------------- residual streams, grouped norm

def embed_positions(table: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor,
                    freqs: Optional[torch.Tensor], out: torch.Tensor, copies: int, precise: bool) -> None:
    """out [T, copies, H] (32-bit) = table[token] + sinusoid(position), the same in every copy.
    ``freqs``: float64 [ceil(H/2)], or None for no position vector."""
    _need_cuda(table, tokens, positions, freqs, out)
    T = tokens.shape[0]
    H = table.shape[1]
    if freqs is not None and (freqs.dtype != torch.float64 or freqs.numel() < (H + 1) // 2):
        raise KernelError("embed_positions: freqs must be float64 [ceil(H/2)]")
    check(library().mf_embed_positions(table.data_ptr(), dtype_code(table), tokens.data_ptr(), positions.data_ptr(),
                                       _ptr(freqs), out.data_ptr(), T, H, copies, int(precise), _stream()),
          "embed_positions")


def hyper_update_norm(streams: torch.Tensor, delta: Optional[torch.Tensor], delta_bias: Optional[torch.Tensor],
                      mix: Optional[torch.Tensor], w_out: Optional[torch.Tensor], w_in: Optional[torch.Tensor],
                      weight: torch.Tensor, eps: float, groups: int, out: torch.Tensor, n_streams: int,
                      rows: Optional[torch.Tensor] = None) -> None:
    """Write ``delta`` back into the streams (``x_t <- sum_s mix[s, t] x_s + w_out[t] (delta + bias)``), read
    them (``u = sum_s w_in[s] x_s``) and normalise ``u`` in ``groups`` groups.  ``streams`` is [T, S * H]
    32-bit; with ``rows`` only those rows are produced and the streams stay as they are."""
    _need_cuda(streams, delta, delta_bias, mix, w_out, w_in, weight, out, rows)
    H = out.shape[-1]
    n = out.shape[0]
    check(library().mf_hyper_update_norm(streams.data_ptr(), _ptr(delta), dtype_code(delta) if delta is not None else
                                         dtype_code(out), _ptr(delta_bias), _ptr(mix), _ptr(w_out), _ptr(w_in),
                                         weight.data_ptr(), eps, groups, out.data_ptr(), dtype_code(out), _ptr(rows),
                                         n, H, n_streams, _stream()), "hyper_update_norm")


# ---------------------------------------------------------------------------- attention with talking heads

def biased_kv_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                    seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int, q_out: torch.Tensor,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int, n_kv: int, dim: int, vdim: int,
                    write_kv: bool) -> None:
    _need_cuda(qkv, bias, positions, seq_of_token, block_table, q_out, k_pool, v_pool)
    check(library().mf_biased_kv_store(qkv.data_ptr(), dtype_code(qkv), _ptr(bias), positions.data_ptr(),
                                       seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                       page_size, q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                       dtype_code(q_out), qkv.shape[0], n_heads, n_kv, dim, vdim, int(write_kv),
                                       _stream()), "biased_kv_store")


def attention_talking(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                      n_heads: int, n_kv: int, dim: int, vdim: int, scale: float, softcap: float,
                      talk: Optional[torch.Tensor], window: int, chunk: int) -> None:
    _need_cuda(q, k_pool, v_pool, out, positions, seq_of_token, block_table, talk)
    check(library().mf_attention_talking(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                         dtype_code(q), q.shape[0], n_heads, n_kv, dim, vdim, positions.data_ptr(),
                                         seq_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                         page_size, scale, softcap, _ptr(talk), window, chunk, _stream()),
          "attention_talking")


# ---------------------------------------------------------------------------- gated delta rule

def delta_prepare(proj: torch.Tensor, conv_w: torch.Tensor, taps: int, state: torch.Tensor, conv_off: int,
                  batch, qkv_out: torch.Tensor, beta_out: torch.Tensor, low: torch.Tensor, n_heads: int, n_kv: int,
                  dim: int, vdim: int) -> None:
    """Convolutions, SiLU and unit norms of the step's projections; the slots' convolution tails move on."""
    _need_cuda(proj, conv_w, state, qkv_out, beta_out, low)
    check(library().mf_delta_prepare(proj.data_ptr(), proj.shape[1], conv_w.data_ptr(), taps, state.data_ptr(),
                                     state.stride(0), conv_off, batch.positions.data_ptr(),
                                     batch.seq_of_token.data_ptr(), batch.seq_q_start.data_ptr(),
                                     batch.seq_q_len.data_ptr(), batch.slots.data_ptr(), qkv_out.data_ptr(),
                                     beta_out.data_ptr(), low.data_ptr(), dtype_code(low), low.shape[1],
                                     proj.shape[0], batch.n_seqs, n_heads, n_kv, dim, vdim, _stream()),
          "delta_prepare", launches=2 if taps > 1 else 1)


def delta_gates(ag: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, n_heads: int, dim: int,
                n_gate: int) -> None:
    _need_cuda(ag, a_log, dt_bias)
    check(library().mf_delta_gates(ag.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), ag.shape[0], n_heads, dim,
                                   n_gate, _stream()), "delta_gates")


def delta_recurrence(qkv: torch.Tensor, beta: torch.Tensor, ag: torch.Tensor, state: torch.Tensor, batch,
                     o_out: torch.Tensor, n_heads: int, n_kv: int, dim: int, vdim: int) -> None:
    _need_cuda(qkv, beta, ag, state, o_out)
    check(library().mf_delta_recurrence(qkv.data_ptr(), beta.data_ptr(), ag.data_ptr(), ag.shape[1], state.data_ptr(),
                                        state.stride(0), batch.seq_q_start.data_ptr(), batch.seq_q_len.data_ptr(),
                                        batch.slots.data_ptr(), o_out.data_ptr(), batch.n_seqs, n_heads, n_kv, dim,
                                        vdim, _stream()), "delta_recurrence")


def delta_output(o: torch.Tensor, gate: torch.Tensor, gate_ld: int, weight: torch.Tensor, eps: float,
                 out: torch.Tensor, n_heads: int, vdim: int, weight_per_head: bool = False) -> None:
    """``gate`` points at the first gate of the first token; rows are ``gate_ld`` floats apart.  ``weight`` is
    [vdim], shared by the heads, or with ``weight_per_head`` [n_heads * vdim]."""
    _need_cuda(o, weight, out)
    check(library().mf_delta_output(o.data_ptr(), gate.data_ptr(), gate_ld, weight.data_ptr(), eps, out.data_ptr(),
                                    dtype_code(out), o.shape[0], n_heads, vdim, int(weight_per_head), _stream()),
          "delta_output")


def delta_gates_ex(decay_in: torch.Tensor, decay_ld: int, per_head: bool, kind: int, c: float,
                   a_log: Optional[torch.Tensor], bias: Optional[torch.Tensor], gate_in: torch.Tensor, gate_ld: int,
                   gate_act: str, ag: torch.Tensor, n_heads: int, dim: int, n_gate: int) -> None:
    """``ag`` [T, n_heads * dim + n_gate] (32-bit): a decay per head and key channel from ``decay_in`` (one number
    per head with ``per_head``, shared by its channels), then the gates from ``gate_in``.  ``kind`` 0:
    ``exp(-exp(a_log_h) softplus(x + bias))``; 1: ``exp(-c sigmoid(x + bias))``.  ``gate_act``: ``"sigmoid"`` or
    ``"silu"``.  The inputs are 32-bit, first element of the first token, rows ``*_ld`` floats apart."""
    _need_cuda(ag, a_log, bias)       # the inputs may be column ranges of wider rows
    check(library().mf_delta_gates_ex(decay_in.data_ptr(), decay_ld, int(per_head), kind, c, _ptr(a_log), _ptr(bias),
                                      gate_in.data_ptr(), gate_ld, {"sigmoid": 0, "silu": 1}[gate_act], ag.data_ptr(),
                                      ag.shape[0], n_heads, dim, n_gate, _stream()), "delta_gates")


def gdelta_prepare(proj: torch.Tensor, a_bias: Optional[torch.Tensor], ops_out: torch.Tensor, low: torch.Tensor,
                   low_off: int, n_heads: int, dim: int) -> None:
    """Operands of the generalized delta rule from ``proj`` [T, r | k | v | a | ...] (32-bit): ``ops_out``
    [T, 4 n_heads dim] gets r | k | unit k | sigmoid(a + a_bias) * unit k; ``low`` [T, rank] gets tanh of the
    columns from ``low_off`` on."""
    _need_cuda(proj, ops_out, low, a_bias)
    check(library().mf_gdelta_prepare(proj.data_ptr(), proj.shape[1], _ptr(a_bias), ops_out.data_ptr(), low.data_ptr(),
                                      dtype_code(low), low_off, low.shape[1], proj.shape[0], n_heads, dim, _stream()),
          "gdelta_prepare")


def gdelta_recurrence(ops_in: torch.Tensor, w: torch.Tensor, w_ld: int, v: torch.Tensor, v_ld: int,
                      state: torch.Tensor, batch, o_out: torch.Tensor, n_heads: int, dim: int) -> None:
    """``S <- diag(w) S - (a u)(u^T S) + k v^T; o = S^T r`` per head from the slot's state, token after token."""
    _need_cuda(ops_in, w, state, o_out)
    check(library().mf_gdelta_recurrence(ops_in.data_ptr(), w.data_ptr(), w_ld, v.data_ptr(), v_ld, state.data_ptr(),
                                         state.stride(0), batch.seq_q_start.data_ptr(), batch.seq_q_len.data_ptr(),
                                         batch.slots.data_ptr(), o_out.data_ptr(), batch.n_seqs, n_heads, dim,
                                         _stream()), "gdelta_recurrence")


# ---------------------------------------------------------------------------- a sublayer's input and its norm

def conv_input(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, tail_off: int, batch, out: torch.Tensor) -> None:
    """``out = x + conv(x)``: ``x`` [T, H] the 32-bit stream, ``w`` [H, taps] (32-bit), the last taps-1 rows of
    every sequence in its slot of ``state`` from float ``tail_off`` on; they move on after they were read."""
    _need_cuda(x, w, state, out)
    T, H = x.shape
    taps = w.shape[1]
    check(library().mf_conv_input(x.data_ptr(), T, H, w.data_ptr(), taps, state.data_ptr(), state.stride(0), tail_off,
                                  batch.seq_of_token.data_ptr(), batch.seq_q_start.data_ptr(),
                                  batch.seq_q_len.data_ptr(), batch.slots.data_ptr(), batch.n_seqs, out.data_ptr(),
                                  dtype_code(out), _stream()), "conv_input",
          launches=2 if taps > 1 and T != batch.n_seqs else 1)


def postnorm_add(x: torch.Tensor, y1: torch.Tensor, s1: float, y2: Optional[torch.Tensor], s2: float,
                 weight: torch.Tensor, eps: float) -> None:
    """``x += rms(s1 y1 + s2 y2) * weight`` on the 32-bit stream ``x`` [T, H]; ``y2`` may be None."""
    _need_cuda(x, y1, y2, weight)
    if y2 is not None and y2.dtype != y1.dtype:
        raise KernelError("postnorm_add: the two branches must have one dtype")
    check(library().mf_postnorm_add(x.data_ptr(), x.shape[0], x.shape[1], y1.data_ptr(), s1, _ptr(y2), s2,
                                    dtype_code(y1), weight.data_ptr(), eps, _stream()), "postnorm_add")


def qk_norm_rope(proj: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_dim: int, rot: int,
                 values_from_keys: bool, eps: float, magnitude: float, bias, q_w, k_w, inv_f, inv_d, vinv_f, vinv_d,
                 batch, block_table: torch.Tensor, page_size: int, q_out: torch.Tensor, k_pool: torch.Tensor,
                 v_pool: torch.Tensor, write_kv: bool) -> None:
    """Biases, the norms of queries and keys over their whole projections, the rotation (cosine and sine times
    ``magnitude``), the values (own, optionally rotated with ``vinv_*``, or the keys as projected) and the cache
    write."""
    _need_cuda(proj, q_out, k_pool, v_pool, bias, q_w, k_w, inv_f, inv_d, vinv_f, vinv_d, block_table)
    check(library().mf_qk_norm_rope(proj.data_ptr(), proj.shape[1], dtype_code(proj), dtype_code(q_out), proj.shape[0], n_heads, n_kv,
                                    head_dim, v_dim, rot, 1 if values_from_keys else 0, eps, magnitude, _ptr(bias),
                                    _ptr(q_w), _ptr(k_w), _ptr(inv_f), _ptr(inv_d), _ptr(vinv_f), _ptr(vinv_d),
                                    batch.positions.data_ptr(), batch.seq_of_token.data_ptr(), block_table.data_ptr(),
                                    block_table.shape[1], page_size, q_out.data_ptr(), k_pool.data_ptr(),
                                    v_pool.data_ptr(), int(write_kv), _stream()), "qk_norm_rope")


def rotate_rows(x: torch.Tensor, n_heads: int, d: int, rot: int, positions: torch.Tensor, inv_f, inv_d,
                sign: float) -> None:
    """The heads of every row of ``x`` [T, n_heads * d] turned in place by ``sign * position`` (half-split pairs
    over the first ``rot`` channels)."""
    _need_cuda(x, positions, inv_f, inv_d)
    check(library().mf_rotate_rows(x.data_ptr(), dtype_code(x), x.shape[0], n_heads, d, rot, positions.data_ptr(),
                                   _ptr(inv_f), _ptr(inv_d), sign, _stream()), "rotate_rows")


# ---------------------------------------------------------------------------- mixture of experts

def moe_route(z: torch.Tensor, n_groups: int, keep: int, top: int, route_scale: float, ids: torch.Tensor,
              weights: torch.Tensor, n_experts: Optional[int] = None, softmax: bool = False,
              bias: Optional[torch.Tensor] = None, renormalize: bool = False) -> None:
    """The router's choice from logits ``z`` [T, >= n_experts] (the first ``n_experts`` columns of every row;
    default all): scores by sigmoid or, with ``softmax``, by a softmax over the experts; ``bias`` (32-bit, one
    per expert) is added for the choice only; ``renormalize``: the chosen weights are divided by their sum."""
    _need_cuda(z, ids, weights, bias)
    E = z.shape[1] if n_experts is None else n_experts
    check(library().mf_moe_route(z.data_ptr(), z.shape[1], z.shape[0], E, n_groups, keep, top, route_scale,
                                 (1 if softmax else 0) | (2 if renormalize else 0), _ptr(bias), ids.data_ptr(),
                                 weights.data_ptr(), _stream()),
          "moe_route")


def moe_rows(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, y: torch.Tensor,
             limit: float, alpha: float, up_offset: float = 1.0, act: Optional[str] = None) -> None:
    """``act`` (an activation without a gate): the experts are ``down(act(up x))`` and ``w_gu`` is [E, 1, ff, H].
    y [T, top, moe_rows_slices(ff), H] (32-bit) = each chosen expert's output for its token, in the
    partial sums of the slices its columns are cut into, not yet weighted.  A choice beyond the stacked
    experts (an identity expert) writes nothing."""
    _need_cuda(x, w_gu, w_down, ids, y)
    T, H = x.shape
    check(library().mf_moe_rows(x.data_ptr(), w_gu.data_ptr(), w_down.data_ptr(), dtype_code(x), ids.data_ptr(),
                                y.data_ptr(), T, H, w_down.shape[2], ids.shape[1], limit, alpha, up_offset,
                                w_down.shape[0], -1 if act is None else activation_code(act), _stream()),
          "moe_rows")


def moe_rows_slices(ff: int) -> int:
    """Partial sums per (token, chosen expert) that ``moe_rows`` writes for experts ``ff`` wide."""
    return int(library().mf_moe_rows_slices(ff))


def moe_combine(y: torch.Tensor, weights: torch.Tensor, slot_of: Optional[torch.Tensor], out: torch.Tensor,
                slices: int = 1, ids: Optional[torch.Tensor] = None, n_real: int = 0,
                x: Optional[torch.Tensor] = None, shared: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.Tensor] = None, gate_ld: int = 0) -> None:
    """The weighted sum of the chosen experts' outputs.  With ``ids``, ``n_real`` and ``x``: a choice from
    ``n_real`` on is an identity expert and contributes ``x[t]``.  With ``shared`` [T, H]: it is added, times
    sigmoid(``shared_gate[t * gate_ld]``) (32-bit logits, e.g. a column of the router's product) where given."""
    _need_cuda(y, weights, slot_of, out, ids, x, shared)
    T, H = out.shape
    for extra in (x, shared):
        if extra is not None and extra.dtype != out.dtype:
            raise KernelError("moe_combine: the input and the shared branch have the output's dtype")
    check(library().mf_moe_combine(y.data_ptr(), dtype_code(y), weights.data_ptr(), _ptr(slot_of), out.data_ptr(),
                                   dtype_code(out), T, H, weights.shape[1], slices, _ptr(ids), n_real, _ptr(x),
                                   _ptr(shared), _ptr(shared_gate), gate_ld, _stream()), "moe_combine")


def attention_talking_tc_ok(n_heads: int, n_kv: int, dim: int, vdim: int, page_size: int) -> bool:
    """Whether the tensor-core kernel for portions of prompts takes these sizes."""
    return bool(library().mf_attention_talking_tc_ok(n_heads, n_kv, dim, vdim, page_size))


def attention_talking_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                         seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_ctx_len: torch.Tensor,
                         table_row0: int, max_q_len: int, block_table: torch.Tensor, page_size: int, n_heads: int,
                         n_kv: int, dim: int, vdim: int, scale: float, softcap: float, talk: Optional[torch.Tensor],
                         window: int, chunk: int, splits: int = 0, part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None, first_row: int = 0) -> None:
    """Talking-heads attention of prompt portions, bfloat16, on the tensor cores.  ``q`` / ``out`` are the
    whole step's rows; the three per-sequence arrays describe the sequences that start at row
    ``table_row0`` of ``block_table``.  ``splits`` > 0 (from ``attention_talking_prefill_splits``): long key
    ranges are cut across blocks and merged; the scratch holds ``T * splits * n_heads * (vdim | 2)`` floats
    and the portions are the step's rows from ``first_row`` on."""
    _need_cuda(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, block_table, talk, part_o, part_ml)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_talking_tc: bfloat16 only")
    T = q.shape[0]
    if splits and (part_o is None or part_ml is None or part_o.numel() < T * splits * n_heads * vdim
                   or part_ml.numel() < T * splits * n_heads * 2):
        raise KernelError("attention_talking_tc: scratch for the splits is missing or too small")
    check(library().mf_attention_talking_tc(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                            seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_ctx_len.data_ptr(),
                                            table_row0, seq_q_len.shape[0], max_q_len, n_heads, n_kv, dim, vdim,
                                            block_table.data_ptr(), block_table.shape[1], page_size, scale, softcap,
                                            _ptr(talk), window, chunk, splits, _ptr(part_o), _ptr(part_ml), first_row,
                                            T - first_row, _stream()), "attention_talking_tc",
          launches=2 if splits else 1)


def attention_talking_prefill_splits(max_keys: int) -> int:
    """Splits for portions of prompts whose queries see at most ``max_keys`` keys (0: not worth cutting)."""
    return int(library().mf_attention_talking_prefill_splits(max_keys))


def attention_talking_splits(max_keys: int) -> int:
    """Key splits of a decode launch when no query sees more than ``max_keys`` keys."""
    return int(library().mf_attention_talking_splits(max_keys))


def attention_talking_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                             seq_q_start: torch.Tensor, seq_q_len: torch.Tensor, seq_ctx_len: torch.Tensor,
                             block_table: torch.Tensor, page_size: int, n_heads: int, n_kv: int, dim: int, vdim: int,
                             scale: float, softcap: float, talk: Optional[torch.Tensor], window: int, chunk: int,
                             splits: int, part_o: torch.Tensor, part_ml: torch.Tensor) -> None:
    """Talking-heads attention of sequences that bring one token each (rows 0.. of the block table),
    bfloat16: the tensor-core kernel over splits of the keys, then the merge of the splits."""
    _need_cuda(q, k_pool, v_pool, out, seq_q_start, seq_q_len, seq_ctx_len, block_table, talk, part_o, part_ml)
    n = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        raise KernelError("attention_talking_decode: bfloat16 only")
    if part_o.numel() < n * splits * n_heads * vdim or part_ml.numel() < n * splits * n_heads * 2:
        raise KernelError("attention_talking_decode: scratch too small")
    check(library().mf_attention_talking_decode(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
                                                seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_ctx_len.data_ptr(),
                                                n, n_heads, n_kv, dim, vdim, block_table.data_ptr(),
                                                block_table.shape[1], page_size, scale, softcap, _ptr(talk), window,
                                                chunk, splits, part_o.data_ptr(), part_ml.data_ptr(), _stream()),
          "attention_talking_decode", launches=2)


def moe_grouped_ok(hidden: int, ff: int, n_experts: int) -> bool:
    """Whether the sorted, tiled expert path takes these sizes."""
    return bool(library().mf_moe_grouped_ok(hidden, ff, n_experts))


def moe_grouped_max_tiles(T: int, top: int, n_experts: int) -> int:
    return int(library().mf_moe_grouped_max_tiles(T, top, n_experts))


def moe_sort(ids: torch.Tensor, n_experts: int, slot_of: torch.Tensor, row_token: torch.Tensor, meta: torch.Tensor,
             tiles: torch.Tensor, ends: Optional[torch.Tensor] = None) -> None:
    """Order the (token, choice) pairs by expert: ``slot_of`` [T * top] the row of every pair, ``row_token``
    the token of every row, ``meta[0]`` the number of tiles, ``tiles`` [n, 3] = expert, first row, rows, and
    (if given) ``ends`` [n_experts] the row at which every expert's range ends."""
    _need_cuda(ids, slot_of, row_token, meta, tiles, ends)
    T, top = ids.shape
    if tiles.numel() < 3 * moe_grouped_max_tiles(T, top, n_experts):
        raise KernelError("moe_sort: the tile list is too small")
    check(library().mf_moe_sort(ids.data_ptr(), T, n_experts, top, slot_of.data_ptr(), row_token.data_ptr(),
                                meta.data_ptr(), tiles.data_ptr(), _ptr(ends), _stream()), "moe_sort")


def moe_gather_rows(x: torch.Tensor, row_token: torch.Tensor, xg: torch.Tensor) -> None:
    """xg[row] = x[row_token[row]] (bfloat16 rows of a multiple of 8 columns)."""
    _need_cuda(x, row_token, xg)
    check(library().mf_moe_gather_rows(x.data_ptr(), row_token.data_ptr(), xg.data_ptr(), xg.shape[0], x.shape[1],
                                       _stream()), "moe_gather_rows")


def moe_activation(gu: torch.Tensor, act: torch.Tensor, limit: float, alpha: float, up_offset: float = 1.0) -> None:
    """act [rows, ff] from a product gu [rows, 2 ff] (gate columns, then up columns): the clamped gated activation."""
    _need_cuda(gu, act)
    check(library().mf_moe_activation(gu.data_ptr(), act.data_ptr(), act.shape[0], act.shape[1], limit, alpha,
                                      up_offset, _stream()), "moe_activation")


def moe_grouped_up(x: torch.Tensor, w_gu: torch.Tensor, row_token: torch.Tensor, meta: torch.Tensor,
                   tiles: torch.Tensor, act: torch.Tensor, top: int, limit: float, alpha: float,
                   up_offset: float = 1.0, ungated: Optional[str] = None) -> None:
    _need_cuda(x, w_gu, row_token, meta, tiles, act)
    T, H = x.shape
    E, _, ff, _ = w_gu.shape
    check(library().mf_moe_grouped_up(x.data_ptr(), w_gu.data_ptr(), row_token.data_ptr(), meta.data_ptr(),
                                      tiles.data_ptr(), act.data_ptr(), T, H, ff, E, top, limit, alpha, up_offset,
                                      -1 if ungated is None else activation_code(ungated), _stream()),
          "moe_grouped_up")


def moe_grouped_down(act: torch.Tensor, w_down: torch.Tensor, meta: torch.Tensor, tiles: torch.Tensor,
                     y: torch.Tensor, T: int, top: int) -> None:
    _need_cuda(act, w_down, meta, tiles, y)
    E, H, ff = w_down.shape
    check(library().mf_moe_grouped_down(act.data_ptr(), w_down.data_ptr(), meta.data_ptr(), tiles.data_ptr(),
                                        y.data_ptr(), T, H, ff, E, top, _stream()), "moe_grouped_down")
