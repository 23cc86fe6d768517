"""Tensor-level entry points of the kernels.

Each function checks nothing twice (the extension validates its arguments) and allocates
only its result, from the caller's device.  Matrix products are library calls
(:func:`linear`), as they are in the reference (``F.linear`` at ampere_kv/runner.py:64-66,
165, 174-177, 297); everything else on the step's path is a kernel of ``_C``.  There is no
fallback: without the extension these functions raise.
"""

from __future__ import annotations

import math
import os

import torch

from . import build

#: query tokens of one sequence that one attention tile covers (the kernels cut it further as they need)
ATTENTION_Q_TILE = 32

_EXT = None

#: kernels of this package launched since the last reset (the benchmark reports it)
launch_count = 0


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


def ext():
    """The loaded extension module (built on first use)."""
    global _EXT
    if _EXT is None:
        _EXT = build.load()
    return _EXT


def smoke_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ext().smoke_add(a, b)


def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor | None = None,
              sampled: torch.Tensor | None = None, scale: float = 1.0, positions: torch.Tensor | None = None,
              position_rows: torch.Tensor | None = None) -> torch.Tensor:
    """float32 residual stream [tokens, hidden] gathered from ``table`` rows, times ``scale``, plus (with
    ``position_rows`` [max positions, hidden] and ``positions``) the row of each token's position.  With
    ``sampled`` (int32, on the device) an id of ``-(r + 1)`` stands for ``sampled[r]``: the token the previous step
    chose in its row r."""
    hidden = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    if scale == 1.0 and position_rows is None:
        ext().embedding(ids, table, hidden, status, sampled)
    else:
        ext().embedding(ids, table, hidden, status, sampled, float(scale), positions, position_rows)
    _launched()
    return hidden


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(logits / cap)`` in place on float32 logits."""
    ext().softcap(logits, float(cap))
    _launched()
    return logits


def add_rmsnorm(hidden: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                status: torch.Tensor | None = None) -> torch.Tensor:
    """``hidden += delta`` in place (whole-batch form), then RMSNorm times ``weight``.

    With ``rows`` only those rows are normalised (``hidden`` is left as it is) and the
    result is [len(rows), hidden].
    """
    n = hidden.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, hidden.shape[1]), dtype=out_dtype, device=hidden.device)
    ext().add_rmsnorm(hidden, delta, weight, out, rows, float(eps), status)
    _launched()
    return out


def add_layernorm(hidden: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                  status: torch.Tensor | None = None) -> torch.Tensor:
    """``hidden += delta`` in place (whole-batch form), then ``(x - mean) / sqrt(var + eps) * weight`` of every row
    (the variance is the mean of the squared deviations).  With ``rows`` only those rows are normalised and
    ``hidden`` is left as it is."""
    n = hidden.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, hidden.shape[1]), dtype=out_dtype, device=hidden.device)
    ext().add_layernorm(hidden, delta, weight, out, rows, float(eps), status)
    _launched()
    return out


class Mirrored:
    """What a block leaves behind when nothing is pending: ``hidden`` holds every sum, and ``copy`` is the same
    stream in the compute dtype (``hidden`` itself when that is float32), ready to be a product's operand."""

    def __init__(self, hidden: torch.Tensor, copy: torch.Tensor):
        self.hidden, self.copy = hidden, copy


class ExpertParts:
    """A routed feed-forward's result before its sum: float32 rows ``parts`` [tokens * top, hidden] (a token's
    ``top`` rows side by side, already weighted) and the shared expert's ``shared`` [tokens, hidden] or None.  A norm
    that knows it adds them up in the kernel that norms them; anyone else calls :meth:`materialize`."""

    def __init__(self, parts: torch.Tensor, shared: torch.Tensor | None, top: int):
        self.parts, self.shared, self.top = parts, shared, int(top)

    def materialize(self) -> torch.Tensor:
        return moe_combine(self.parts, self.shared, top=self.top)


def branch_layernorm(hidden: torch.Tensor, branch, weight: torch.Tensor, eps: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``hidden += (branch - mean) / sqrt(var + eps) * weight`` in place, row by row in float32 (``branch`` in the
    compute dtype or float32, or an :class:`ExpertParts`).  Returns the new ``hidden`` in ``out_dtype``: a rounded
    copy, or ``hidden`` itself when ``out_dtype`` is float32."""
    copy = None if out_dtype == torch.float32 else torch.empty(hidden.shape, dtype=out_dtype, device=hidden.device)
    if isinstance(branch, ExpertParts):
        ext().branch_layernorm_parts(hidden, branch.parts, branch.shared, weight, copy, float(eps), branch.top)
        _launched()
        return hidden if copy is None else copy
    ext().branch_layernorm(hidden, branch, weight, copy, float(eps))
    _launched()
    return hidden if copy is None else copy


def stream_copy(hidden: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream as a product's operand: itself, or its rounding to ``dtype``."""
    if dtype == torch.float32:
        return hidden
    out = torch.empty(hidden.shape, dtype=dtype, device=hidden.device)
    ext().stream_copy(hidden, out)
    _launched()
    return out


GLU_KINDS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def glu(gate_up: torch.Tensor, kind: str, block: int = 0, limit: float = 0.0, slope: float = 1.0) -> torch.Tensor:
    """``act(gate) * up`` of [tokens, 2 * intermediate]; gate and up columns alternate in runs of ``block`` columns
    (0: all gate columns first).  ``kind``: ``"silu"``, ``"gelu_tanh"``, or ``"clamped_swish"``:
    ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``g * sigmoid(slope * g) * (u + 1)``."""
    out = torch.empty((gate_up.shape[0], gate_up.shape[1] // 2), dtype=gate_up.dtype, device=gate_up.device)
    ext().glu(gate_up, out, GLU_KINDS[kind], int(block), float(limit), float(slope))
    _launched()
    return out


GATE_UP_RUN = 64   # gate and up rows alternate in runs of this many when one GEMM tile is to hold both


def silu_mul(gate_up: torch.Tensor, out_dtype: torch.dtype | None = None, block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` of [tokens, 2 * intermediate].  Gate and up columns alternate in runs of ``block``
    columns (0: all gate columns first).  A 3-D float32 input is a stack of split-K partial sums that are added
    up first; then ``out_dtype`` names the result's type."""
    if gate_up.dim() == 3:
        out_dtype = out_dtype or torch.bfloat16
    else:
        out_dtype = gate_up.dtype
    out = torch.empty((gate_up.shape[-2], gate_up.shape[-1] // 2), dtype=out_dtype, device=gate_up.device)
    ext().silu_mul(gate_up, out, int(block))
    _launched()
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """One matrix [2 * intermediate, k] whose rows are ``block`` gate rows, then the ``block`` up rows of the same
    outputs, and so on."""
    inter, k = gate.shape
    return torch.stack((gate.view(inter // block, block, k), up.view(inter // block, block, k)), dim=1).reshape(2 * inter, k)


def gated_linear(x: torch.Tensor, gate_up: torch.Tensor, block: int, status: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` with gate and up rows stored in alternating runs of ``block`` (0: all gate
    rows first).  Few bfloat16 tokens and ``block == GATE_UP_RUN``: one tcgen05 kernel that applies the activation
    to its output tile; otherwise the product and the activation kernel."""
    x, normed, small = _operand(x, gate_up)
    if block == GATE_UP_RUN and small and gate_up.shape[0] % 128 == 0:
        return small_m_gemm(x, gate_up, status=status, gated=True, normed=normed)
    if normed:
        return silu_mul(small_m_gemm(None, gate_up, status=status, normed=normed), torch.bfloat16, block)
    return silu_mul(linear(x, gate_up, partial_ok=True, status=status), x.dtype, block)


def qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache, *, num_heads,
                       num_kv_heads, head_dim, rotary_dim, eps, want_kv: bool = False, status=None):
    """Per-head RMSNorm of q and k, rotation by position, K/V written to their cache slots.

    Returns q [tokens, heads * head_dim] (and the dense k, v when ``want_kv``).
    """
    n = qkv.shape[-2]
    out_dtype = torch.bfloat16 if qkv.dim() == 3 else qkv.dtype      # 3-D: float32 split-K partial sums
    q_out = torch.empty((n, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
    k_out = v_out = None
    if want_kv:
        k_out = torch.empty((n, num_kv_heads * head_dim), dtype=out_dtype, device=qkv.device)
        v_out = torch.empty_like(k_out)
    ext().qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, q_out, k_out, v_out, k_cache,
                             v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, float(eps), status)
    _launched()
    return (q_out, k_out, v_out) if want_kv else q_out


def project_qkv(x, w_qkv, bias, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache, *, num_heads,
                num_kv_heads, head_dim, rotary_dim, eps, status=None):
    """The q/k/v projection of ``x``, then per-head RMSNorm of q and k, rotation of the first ``rotary_dim`` dims
    by position, and K/V written to their cache slots.  Returns q [tokens, heads * head_dim].

    Few bfloat16 tokens with heads of 128 dims that are rotated whole: one tcgen05 kernel whose 128-row tile is
    one head and does all of it on the tile.  Otherwise the product, then ``qk_norm_rope_write``.
    """
    on_tile = (bias is None and head_dim == 128 and (inv_freq is None or rotary_dim == 128)
               and w_qkv.shape[0] == (num_heads + 2 * num_kv_heads) * 128)
    if on_tile:
        x, normed, small = _operand(x, w_qkv)
        if small:
            q_out = torch.empty((positions.shape[0], num_heads * 128), dtype=torch.bfloat16, device=w_qkv.device)
            ext().small_m_gemm_qkv(x, w_qkv, q_out, positions, slots, q_weight, k_weight, inv_freq, k_cache,
                                   v_cache, num_heads, num_kv_heads, float(eps), _cluster_splits(w_qkv), status,
                                   **normed)
            _launched()
            return q_out
    qkv = linear(x, w_qkv, bias, partial_ok=True, status=status)
    return qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache,
                              num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                              rotary_dim=rotary_dim, eps=eps, status=status)


def kv_write(k, v, slots, k_cache, v_cache, status=None) -> None:
    ext().kv_write(k, v, slots, k_cache, v_cache, status)
    _launched()


#: streaming multiprocessors assumed when no device can be asked (planning on a host without a GPU): a B200's
FALLBACK_SM_COUNT = 148
_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked once per device."""
    if not torch.cuda.is_available():
        return FALLBACK_SM_COUNT
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNT[index]


def attention_q_tile(head_dim: int, group_size: int) -> int:
    """Query tokens per attention tile that suit a mixer of this shape: the tcgen05 prompt kernel's CTAs take
    128 // group tokens (128 rows), so a group that does not divide 128 gets tiles of exactly that many."""
    if head_dim == 128 and 1 <= group_size <= 16 and 128 % group_size:
        return 128 // group_size
    return ATTENTION_Q_TILE


def attention_takes_tensor_cores(dtype: torch.dtype, head_dim: int, group_size: int, page_size: int) -> bool:
    """Whether the TMA + tensor-core attention kernels take these sizes (else the general kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group_size <= 16 and page_size >= 8
            and page_size & (page_size - 1) == 0)


def choose_splits(num_tiles: int, num_kv_heads: int, rows_per_tile: int, max_context: int,
                  tensor_core: bool = False, mean_context: int | None = None, sms: int | None = None) -> int:
    """How many key ranges each decoded token's attention is cut into so that a small batch still fills the GPU
    and a long sequence among short ones does not keep one CTA walking alone.  ``max_context`` / ``mean_context``:
    the keys the longest and the average token of the batch walks (the mean defaults to the maximum).

    The tensor-core decode kernel runs one CTA per (token, kv head, split), four to an SM; the general kernel
    one warp per (token, kv head, 8 rows, split), sixteen to an SM.
    """
    sms = sms or sm_count()
    if tensor_core:
        # 1, 2, 4 or 8 splits (merged inside the kernel by a cluster).  A cost in microseconds, fitted to
        # measurements on B200 (32 q-heads, 8 kv-heads, head size 128, batches of 4 to 64, 1,088 to 8,000 keys,
        # equal and mixed lengths): a CTA spends about 1.1 us on a 32-key block and a fixed 5.5 us (7.5 us in a
        # cluster) on start-up and merge; the GPU holds four CTAs per SM at a time.  With equal lengths all CTAs end
        # together, so a grid that needs a further round of CTAs pays for a whole one; with mixed lengths slots
        # free up all the time and only the fraction counts.  The longest sequences' CTAs start first (the batch
        # layout orders the tiles so), so the step takes the longest walk or the rounds of mean walks, whichever
        # is more, and never less than the bytes need to cross the memory system.
        # Measured (us at 1/2/4/8 splits): batch 8 at 1,088 keys 35/24/15/12; batch 24: 40/27/32/36; batch 64:
        # 48/57/68/95; batch 48 at 4,096 keys 169/172/142/159; batch 64 with 300 to 4,600 keys (mean 2,500):
        # 171/110/119/144; batch 40 likewise: 160/94/75/88; batch 20: 144/81/48/46.
        items, slots = max(1, num_tiles * num_kv_heads), sms * 4
        blocks_max = max(1, (max_context + 31) // 32)
        blocks_mean = blocks_max if mean_context is None else max(1, min(blocks_max, (int(mean_context) + 31) // 32))
        evenness = (blocks_mean / blocks_max) ** 2
        moved = items * blocks_mean * 16384 / 6.0e6       # us for the K/V bytes (heads of 128 dims) at 6 TB/s
        best, best_cost = 1, None
        for i, s in enumerate((1, 2, 4, 8)):
            if s > 1 and blocks_max // s < 2:
                break
            fixed = 5.5 if s == 1 else 7.5
            walk_max = -(-blocks_max // s) * 1.1 + fixed
            walk_mean = -(-blocks_mean // s) * 1.1 + fixed
            rounds = items * s / slots
            rounds += (math.ceil(rounds) - rounds) * evenness
            cost = max(walk_max, rounds * walk_mean, moved) * (1.0 + 0.03 * i)
            if best_cost is None or cost < best_cost:
                best, best_cost = s, cost
        return best
    items, target, min_keys = max(1, num_tiles * num_kv_heads * ((rows_per_tile + 7) // 8)), sms * 16, 128
    if items >= target or max_context <= min_keys:
        return 1
    want = target // items
    return int(max(1, min(want, (max_context + min_keys - 1) // min_keys, 64)))


def paged_attention(q, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq, *, num_tiles,
                    q_tile, num_splits, num_heads, num_kv_heads, window, scale, partials=None, status=None,
                    kernel: str = "auto", out=None):
    """Causal attention of the batch's new tokens over the paged cache.  ``kernel``: ``"auto"`` takes the
    tensor-core kernels where they fit (bfloat16, head size 64 or 128; prompt portions at head size 128 and groups
    of up to 16 q-heads on tcgen05) and the general kernel elsewhere; ``"general"`` forces the latter, ``"mma"``
    keeps prompt portions on the mma.sync kernel, ``"tcgen05-narrow"`` / ``"tcgen05-wide"`` pick the form of the
    tcgen05 prompt kernel that the grid's size otherwise decides.  Only the rows of the given tiles are written; with ``out`` they
    go into that tensor (a batch may be covered by two calls with different tile sizes)."""
    if out is None:
        out = torch.empty_like(q)
    if num_splits > 1 and partials is None:
        head_dim = q.shape[1] // num_heads
        partials = torch.empty((q.shape[0] * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32,
                               device=q.device)
    ext().paged_attention(q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq,
                          partials, num_tiles, q_tile, num_splits, num_heads, num_kv_heads, int(window or 0),
                          float(scale), status, {"auto": 0, "general": 1, "mma": 2, "tcgen05-narrow": 3, "tcgen05-wide": 4}[kernel])
    _launched(2 if num_splits > 1 else 1)
    return out


def scored_takes_tensor_cores(dtype: torch.dtype, head_dim: int, v_dim: int, group_size: int, page_size: int,
                              prompt: bool) -> bool:
    """Whether the tensor-core kernels' scored forms take these sizes: bfloat16 keys and values of the same width in
    storage of their own; prompt tiles at 128 dims on the tcgen05 kernel, single tokens at 64 or 128 dims on the
    TMA + mma.sync decode kernel (1, 2, 4 or 8 key splits).  Everything else runs on the general kernel."""
    if dtype != torch.bfloat16 or head_dim != v_dim or not 1 <= group_size <= 16 or page_size & (page_size - 1):
        return False
    return (head_dim == 128 and page_size >= 16) if prompt else (head_dim in (64, 128) and page_size >= 8)


def shared_rows_take_tensor_cores(dtype: torch.dtype, row: int, v_dim: int) -> bool:
    """Whether the mma.sync kernel for rows that are key and value at once takes these sizes (bfloat16, a key width
    that is a multiple of 16 up to 576, a value width of 64, 128, 256 or 512)."""
    return dtype == torch.bfloat16 and row % 16 == 0 and 16 <= row <= 576 and v_dim in (64, 128, 256, 512) \
        and v_dim <= row


def choose_splits_shared_rows(num_tiles: int, num_kv_heads: int, rows_per_tile: int, max_context: int,
                              sms: int | None = None) -> int:
    """Key splits for the shared-row kernel: a CTA per (tile, kv head, 16 rows, split), two to an SM; a split walks
    at least 128 keys (every split writes a partial row of the value width per head, and a merge reads them)."""
    sms = sms or sm_count()
    items = max(1, num_tiles * num_kv_heads * ((rows_per_tile + 15) // 16))
    if items >= 2 * sms or max_context <= 256:
        return 1
    return int(max(1, min(2 * sms // items, (max_context + 127) // 128, 32)))


def scored_attention(q, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq, *, num_tiles,
                     q_tile, num_splits, num_heads, num_kv_heads, v_dim, scale, window=0, chunk=0, softcap=0.0,
                     slopes=None, gate=None, partials=None, status=None, out=None, kernel: str = "auto",
                     keep_first: int = 0, sigmoid_weights: bool = False, head_bias=None, out_scale: float = 1.0):
    """Causal attention of the batch's new tokens over paged keys and values of different widths, with the score
    reshaped before the softmax: ``softcap * tanh(score / softcap)`` (``softcap`` > 0), less ``slopes[h]`` times the
    distance to the key (``slopes`` float32 [heads]); a query sees the last ``window`` keys (``window`` > 0) of its own
    block of ``chunk`` positions (``chunk`` > 0), and with ``keep_first`` the keys at positions below it behind the
    window too; ``gate`` (float32 [tokens, heads]) scales each head's output and ``out_scale`` all of them.  With
    ``sigmoid_weights`` there is no softmax: a visible key weighs ``sigmoid(score + head_bias[h])``.
    ``k_cache`` / ``v_cache``: [pages, kv heads, page size, width]; they may be one tensor whose rows are read whole
    as keys and in their first ``v_dim`` elements as values.  Returns [tokens, heads * v_dim]; only the rows of the
    given tiles are written.  ``kernel``: ``"auto"`` takes the tensor-core kernels where they fit
    (:func:`scored_takes_tensor_cores`), ``"general"`` keeps the general kernel."""
    if out is None:
        out = torch.empty((q.shape[0], num_heads * v_dim), dtype=q.dtype, device=q.device)
    if num_splits > 1 and partials is None:
        partials = torch.empty((q.shape[0] * num_heads * num_splits * (v_dim + 2),), dtype=torch.float32,
                               device=q.device)
    ext().scored_attention(q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq, partials,
                           num_tiles, q_tile, num_splits, num_heads, num_kv_heads, int(v_dim), int(window or 0),
                           int(chunk or 0), float(scale), float(softcap or 0.0), slopes, gate, status,
                           {"auto": 0, "general": 1}[kernel], int(keep_first or 0), bool(sigmoid_weights), head_bias,
                           float(out_scale))
    _launched(2 if num_splits > 1 else 1)
    return out


def head_prep(x, slots, k_cache, v_cache, *, num_heads, num_kv_heads, head_dim, v_dim, unit_norm, eps, gated,
              v_keep=None, v_other=None, blend_weight=None, q_weight=None, k_weight=None, has_kv=True, status=None):
    """From one product ``x`` [tokens, q heads | k heads | v heads | a gate column per q head]: q (and k) heads
    scaled to unit RMS and multiplied by ``q_weight`` / ``k_weight`` (float32 [head_dim]) where given,
    ``v <- (1 - blend_weight) v + blend_weight v_other``, k and v written to their cache slots;
    ``v_keep`` receives the layer's own values before the blend.  Without ``has_kv`` the product holds no k and v
    columns.  Returns (q [tokens, heads * head_dim], sigmoid of
    the gate columns as float32 [tokens, heads], or None without ``gated``)."""
    n = x.shape[0]
    q_out = torch.empty((n, num_heads * head_dim), dtype=x.dtype, device=x.device)
    gate = torch.empty((n, num_heads), dtype=torch.float32, device=x.device) if gated else None
    if q_weight is None and k_weight is None and has_kv:
        ext().head_prep(x, slots, q_out, k_cache, v_cache, v_keep, v_other, blend_weight, gate, num_heads,
                        num_kv_heads, head_dim, v_dim, bool(unit_norm), float(eps), status)
    else:
        ext().head_prep(x, slots, q_out, k_cache, v_cache, v_keep, v_other, blend_weight, gate, num_heads,
                        num_kv_heads, head_dim, v_dim, bool(unit_norm), float(eps), status, q_weight, k_weight,
                        bool(has_kv))
    _launched()
    return q_out, gate


def latent_prep(x, positions, slots, q_weight, kv_weight, inv_freq, cache, *, q_rank, kv_rank, rot_dim, rotary_dims,
                eps, status=None):
    """From one product ``x`` [tokens, query latent | key/value latent | rotated key part]: both latents through an
    RMS norm with a plain weight, neighbouring pairs of the rotated part turned by position; the key/value latent
    and the rotated part land side by side in the token's row of ``cache``.  Returns the query latent."""
    q_latent = torch.empty((x.shape[0], q_rank), dtype=x.dtype, device=x.device)
    ext().latent_prep(x, positions, slots, q_weight, kv_weight, inv_freq, q_latent, cache, q_rank, kv_rank, rot_dim,
                      rotary_dims, float(eps), status)
    _launched()
    return q_latent


def rotate_pairs(x, out, positions, inv_freq, *, heads, cols, rotary_dims, in_offset, out_offset) -> None:
    """``out[t, h, out_offset + c] = x[t, h, in_offset + c]`` for ``c < cols``, dims 2i and 2i + 1 of the range
    turned by ``positions[t] * inv_freq[i]`` while they lie in the first ``rotary_dims``."""
    ext().rotate_pairs(x, out, positions, inv_freq, heads, cols, rotary_dims, in_offset, out_offset)
    _launched()


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def linear_activation(x, weight: torch.Tensor, kind: str, status: torch.Tensor | None = None) -> torch.Tensor:
    """``activation(x @ weight.T)``, the activation applied to the product as it is stored (rounded to the compute
    dtype).  Few bfloat16 tokens: one launch of the small-batch product kernel, whose output tile goes through the
    activation; otherwise the library product and the activation kernel.  ``x`` may be a ``LazyNorm``."""
    x, normed, small = _operand(x, weight)
    if small:
        return small_m_gemm(x, weight, status=status, normed=normed, activation=kind)
    return activation(torch.nn.functional.linear(x, weight), kind)


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """``relu(x) ** 2`` (``"relu2"``), the tanh form of GELU (``"gelu_tanh"``) or SiLU, element by element."""
    out = torch.empty_like(x)
    ext().activation(x, out, ACTIVATIONS[kind])
    _launched()
    return out


# ----------------------------------------------------------------------------- the gated delta rule

#: what the delta-rule kernels take: q/k width, value width (a block holds a value column per thread group), taps
DELTA_MAX_DIM = 256
DELTA_MAX_VDIM = 256
DELTA_MAX_TAPS = 16


def delta_shape(head_dim: int, v_dim: int) -> tuple[int, int] | None:
    """(elements of a value column per lane, lanes per column) of the scan kernel for a head of these sizes, or None
    when it does not take them: the smallest of 4, 8, 16, 32 elements with which at most 8 lanes cover the q/k width."""
    if not (0 < head_dim <= DELTA_MAX_DIM and 0 < v_dim <= DELTA_MAX_VDIM):
        return None
    for per_lane in (4, 8, 16, 32):
        lanes = 1
        while lanes * per_lane < head_dim:
            lanes *= 2
        if lanes <= 8:
            return per_lane, lanes
    return None


def delta_state_floats(num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, taps: int) -> tuple[int, int]:
    """(floats of all heads' memory, floats of a request's whole state) as the delta-rule kernels lay a state slot
    out: every head's memory in the scan kernel's own order (the q/k width padded to lanes times elements per lane),
    then the last ``taps - 1`` inputs of the convolutions' channels, rounded up to a multiple of four floats."""
    per_lane, lanes = delta_shape(head_dim, v_dim)
    memory = num_heads * v_dim * lanes * per_lane
    channels = 2 * num_kv_heads * head_dim + num_heads * v_dim
    return memory, (memory + (taps - 1) * channels + 3) // 4 * 4


def delta_prep(x, conv, rate_log, step_bias, state, cu_q, state_slots, *, num_heads, num_kv_heads, head_dim, v_dim,
               taps, unit_eps):
    """From one product ``x`` [tokens, q | k | v | gate | beta | step] (``num_kv_heads`` heads of ``head_dim`` for q
    and k, ``num_heads`` of ``v_dim`` for v and gate, a column per head for beta and step): q, k and v through their
    causal convolutions over the sequence's own earlier tokens (``conv`` float32 [channels, taps], last tap the
    current token's; before the step's first token the inputs come from ``state[slot, memory:]``, zeros at a
    sequence's start) and SiLU; q and k scaled to unit length (q also by ``head_dim ** -0.5``);
    ``beta = sigmoid(.)``, ``decay = exp(-exp(rate_log) * softplus(step + step_bias))``.  ``cu_q`` [sequences + 1]
    gives each sequence's rows, ``state_slots`` its slot (negative: a padded sequence, left alone).  Returns
    (float32 [tokens, q | k | v], float32 [tokens, beta per head | decay per head]).  The state is not changed."""
    n = x.shape[0]
    channels = 2 * num_kv_heads * head_dim + num_heads * v_dim
    qkv = torch.empty((n, channels), dtype=torch.float32, device=x.device)
    coef = torch.empty((n, 2 * num_heads), dtype=torch.float32, device=x.device)
    ext().delta_prep(x, conv, rate_log, step_bias, state, cu_q, state_slots, qkv, coef, num_heads, num_kv_heads,
                     head_dim, v_dim, taps, float(unit_eps))
    _launched()
    return qkv, coef


def delta_scan(qkv, coef, x, norm_weight, state, cu_q, state_slots, *, num_heads, num_kv_heads, head_dim, v_dim, taps,
               norm_eps):
    """The recurrence over the step's tokens, sequence by sequence and head by head, from and into ``state``
    [slots, delta_state_floats(...)[1]] float32: ``S *= decay; u = beta (v - S^T k);
    S += k u^T; o = S^T q``; then ``o / sqrt(mean(o^2) + norm_eps) * norm_weight * silu(gate)`` with the gate columns
    of ``x``.  Also moves the sequence's last ``taps - 1`` convolution inputs (columns of ``x``) into the state.
    Returns [tokens, heads * v_dim] in the dtype of ``x``."""
    out = torch.empty((x.shape[0], num_heads * v_dim), dtype=x.dtype, device=x.device)
    scratch = torch.empty((x.shape[0], num_heads * v_dim), dtype=torch.float32, device=x.device)
    ext().delta_scan(qkv, coef, x, norm_weight, state, cu_q, state_slots, scratch, out, num_heads, num_kv_heads,
                     head_dim, v_dim, taps, float(norm_eps))
    _launched(2)        # the scan; the output norm and the convolutions' memory
    return out


# ----------------------------------------------------------------------------- routed experts

MOE_MAX_EXPERTS = 512
MOE_MAX_TOP = 32
MOE_FORMS = {"auto": 0, "plain": 1, "mma": 2, "few": 3}


#: steps of at most this many tokens compute the router's logits with a warp per (token, expert); the library's
#: product of so few rows with a matrix of a few dozen rows runs on one or two SMs
MOE_ROUTER_TOKENS = 64


def moe_router_logits(x, w_router, status=None):
    """float32 ``x @ w_router.T`` [tokens, experts], accumulated in float32 whatever the operands' dtype."""
    if x.shape[0] <= MOE_ROUTER_TOKENS:
        logits = torch.empty((x.shape[0], w_router.shape[0]), dtype=torch.float32, device=x.device)
        ext().moe_router(x, w_router, logits)
        _launched()
        return logits
    return linear(x, w_router, out_dtype=torch.float32, status=status)


MOE_SCORES = {"sigmoid": 0, "softmax": 1}


def moe_route(logits, correction, *, top, groups, keep_groups, group_top, scale, weight_eps, score: str = "sigmoid"):
    """Scores ``sigmoid(logits)``, or with ``score="softmax"`` the softmax over all experts (float32
    [tokens, experts]); choice scores are the scores plus ``correction``
    (float32 [experts] or None); experts form ``groups`` equal runs, a group's score is the sum of its ``group_top``
    largest choice scores, experts outside the ``keep_groups`` best groups cannot be chosen; the ``top`` largest
    remaining choice scores are chosen (ties: the lower index).  Returns (int32 [tokens, top], float32 [tokens, top]:
    the chosen scores divided by their sum plus ``weight_eps``, times ``scale``)."""
    n = logits.shape[0]
    chosen = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    ext().moe_route(logits, correction, chosen, weights, groups, keep_groups, group_top, float(scale), float(weight_eps),
                    MOE_SCORES[score])
    _launched()
    return chosen, weights


def moe_sort(chosen, experts: int):
    """The (token, choice) pairs in the order of their expert: ``order`` int32 [tokens * top] holds
    ``token * top + choice``, ``offsets`` int32 [experts + 1] where each expert's run begins."""
    order = torch.empty((chosen.numel(),), dtype=torch.int32, device=chosen.device)
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=chosen.device)
    ext().moe_sort(chosen, order, offsets)
    _launched()
    return order, offsets


def moe_gate_up(x, w_gate_up, order, offsets, *, top, limit, slope, kernel: str = "auto", up_offset: float = 1.0):
    """Row r of the result belongs to pair ``order[r]`` and is its expert's ``g * sigmoid(slope * g) * (u + up_offset)``
    with ``g = min(W_gate x, limit)``, ``u = clamp(W_up x, -limit, limit)`` for the pair's token (an infinite limit, a
    slope of one and no offset make it ``silu(g) * u``);
    ``w_gate_up`` [experts, gate rows then up rows, hidden].  [tokens * top, intermediate] in the dtype of ``x``.
    ``kernel``: ``"auto"``: for bfloat16 with a hidden size that is a multiple of eight, the few-rows form (weights
    streamed once, no staging) for the gated product of steps of up to 128 pairs and the tensor cores (``mma.sync``
    tiles) otherwise;
    ``"plain"`` keeps the float-arithmetic form, which is also all of float32; ``"mma"`` / ``"few"`` force one."""
    inter = w_gate_up.shape[1] // 2
    act = torch.empty((order.numel(), inter), dtype=x.dtype, device=x.device)
    ext().moe_gate_up(x, w_gate_up, order, offsets, act, top, float(limit), float(slope), MOE_FORMS[kernel],
                      float(up_offset))
    _launched()
    return act


def moe_down(act, w_down, order, offsets, weights, kernel: str = "auto"):
    """``weights[pair] * W_down[expert] act[r]`` for every sorted row r, written to row ``order[r]`` of a float32
    [tokens * top, hidden].  ``kernel`` as for :func:`moe_gate_up`."""
    out = torch.empty((order.numel(), w_down.shape[1]), dtype=torch.float32, device=act.device)
    ext().moe_down(act, w_down, order, offsets, weights, out, MOE_FORMS[kernel])
    _launched()
    return out


def moe_combine(parts, shared, *, top):
    """``sum over a token's choices of parts[token * top + choice] (+ shared[token])`` in that order, float32
    [tokens, hidden]."""
    out = torch.empty((parts.shape[0] // top, parts.shape[1]), dtype=torch.float32, device=parts.device)
    ext().moe_combine(parts, shared, out, top)
    _launched()
    return out


_SAMPLE_TICKETS: dict = {}      # per device: zeroed row counters of the sampling kernel (it leaves them zero)


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """int32 token per row: the arg-max where ``temperature`` is 0, else the inverse-CDF draw of
    ``softmax(logits / temperature)`` at ``uniform``.  With ``out`` (int32, contiguous, at least a row each) the
    tokens are written there."""
    rows = logits.shape[0]
    if out is None:
        tokens = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        if out.dtype != torch.int32 or out.device != logits.device or out.dim() != 1 or out.shape[0] < rows \
                or not out.is_contiguous():
            raise ValueError("sample: out must be a contiguous int32 vector on the logits' device with a row each")
        tokens = out[:rows]
    tickets = _SAMPLE_TICKETS.get(logits.device)
    if tickets is None or tickets.numel() < rows:
        tickets = torch.zeros((max(rows, 512),), dtype=torch.int32, device=logits.device)
        _SAMPLE_TICKETS[logits.device] = tickets
    parts = torch.empty((4 * rows * ext().sample_slices(),), dtype=torch.float32, device=logits.device)
    ext().sample(logits, temperature, uniform, tokens, parts, tickets)
    _launched()
    return tokens


class Summed:
    """What a product leaves behind when it has added its result to the residual stream itself
    (``linear_into_residual``): ``hidden`` holds the sum already, and ``ssq`` [tiles, tokens] the sums of squares
    of its new values per 128-feature tile, from which the next RMS norm needs no pass over ``hidden``."""

    def __init__(self, hidden: torch.Tensor, ssq: torch.Tensor):
        self.hidden, self.ssq = hidden, ssq


class LazyNorm:
    """An RMS norm that is not computed yet: ``hidden * rsqrt(mean(hidden^2) + eps) * weight`` with the sums of
    squares already known (``Summed``).  ``linear``, ``gated_linear`` and ``project_qkv`` take it in place of a
    tensor and let the small-batch product kernel apply it to its token operand; ``materialize`` runs the norm
    kernel."""

    def __init__(self, summed: Summed, weight: torch.Tensor, eps: float, dtype: torch.dtype, status=None):
        self.hidden, self.ssq, self.weight, self.eps, self.dtype, self.status = (
            summed.hidden, summed.ssq, weight, float(eps), dtype, status)

    @property
    def shape(self):
        return self.hidden.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.hidden, None, self.weight, self.eps, self.dtype, status=self.status)


def _operand(x, weight: torch.Tensor):
    """(tensor or None, normed-x keyword arguments of the extension, fused?) for a token operand that may be a
    ``LazyNorm``.  A lazy norm that the small-batch kernel cannot take is materialized."""
    if not isinstance(x, LazyNorm):
        return x, {}, _takes_small_m(x, weight)
    h = x.hidden
    fused = (use_small_m_gemm and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and h.is_cuda
             and h.shape[0] <= SMALL_M_LIMIT and h.is_contiguous() and weight.is_contiguous()
             and h.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.weight.data_ptr() % 16 == 0
             and h.shape[1] == weight.shape[1]
             and ext().small_m_gemm_supported(h.shape[0], weight.shape[0], weight.shape[1]))
    if not fused:
        t = x.materialize()
        return t, {}, _takes_small_m(t, weight)
    return None, {"nx_hidden": h, "nx_ssq": x.ssq, "nx_weight": x.weight, "nx_eps": x.eps}, True


#: products of at most this many bfloat16 tokens go through the package's own tcgen05 kernel: all it takes.
#: Measured per decode step on B200 against the library product with the row-wise kernels around it: 5.08 against
#: 5.21 ms at 40 tokens, 5.21 against 5.36 ms at 56, 5.17 against 5.37 ms at 64.
SMALL_M_LIMIT = 64
use_small_m_gemm = True
#: up to this many tokens a decode branch adds to the residual stream inside its last product and the next product
#: applies the norm to its own token operand.  Every CTA of that product re-reads the float32 stream for its K
#: range, which grows with the tokens: measured per decode step on B200 against the norm as a kernel of its own,
#: 3.64 against 3.67 ms at 12 tokens, 3.71 against 3.76 ms at 16, but 4.98 against 4.25 ms at 32 and 7.0 against
#: 5.2 ms at 64.
LAZY_NORM_LIMIT = 16
#: hand split-K partial sums to the consuming kernel instead of adding them up inside the product kernel
prefer_partials = False


def _cluster_splits(weight: torch.Tensor) -> int:
    splits = min(ext().small_m_gemm_splits(weight.shape[0], weight.shape[1]), (weight.shape[1] + 63) // 64)
    while splits not in (1, 2, 4, 8):
        splits -= 1
    return splits


def small_m_gemm(x: torch.Tensor | None, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 splits: int | None = None, parts: bool = False, status: torch.Tensor | None = None,
                 gated: bool = False, normed: dict | None = None, activation: str | None = None) -> torch.Tensor:
    """``x @ weight.T`` for 1..64 bfloat16 tokens on the tcgen05 tensor cores, K cut into ``splits`` ranges.

    Default: [tokens, features] in ``out_dtype`` (float32 or bfloat16); the splits (1, 2, 4 or 8 CTAs of a
    cluster) add their float32 partial tiles up through distributed shared memory.  ``parts=True``: the float32
    partial sums themselves, [splits, tokens, features], for a consumer kernel that adds them up.
    ``gated=True``: ``weight`` holds gate and up rows in alternating runs of 64 and the result is
    ``silu(gate) * up``, [tokens, features / 2] bfloat16.  ``normed`` (with ``x`` None): the kernel makes its token
    operand from a residual stream and its sums of squares (``LazyNorm``).  ``activation`` (a name of
    ``ACTIVATIONS``; bfloat16 result only): applied to the product, rounded to bfloat16 first, before it is stored.
    """
    normed = normed or {}
    tokens = x.shape[0] if x is not None else normed["nx_hidden"].shape[0]
    kb_total = (weight.shape[1] + 63) // 64
    if splits is None:
        splits = ext().small_m_gemm_splits(weight.shape[0], weight.shape[1])
    splits = max(1, min(int(splits), kb_total))
    if parts:
        out = torch.empty((splits, tokens, weight.shape[0]), dtype=torch.float32, device=weight.device)
    else:
        while splits not in (1, 2, 4, 8):
            splits -= 1
        out = torch.empty((tokens, weight.shape[0] // 2 if gated else weight.shape[0]),
                          dtype=torch.bfloat16 if gated else out_dtype, device=weight.device)
    if activation is not None:
        ext().small_m_gemm(x, weight, out, splits, status, gated, activation=ACTIVATIONS[activation], **normed)
    else:
        ext().small_m_gemm(x, weight, out, splits, status, gated, **normed)
    _launched()
    return out


def linear_into_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor,
                         status: torch.Tensor | None = None) -> Summed | None:
    """``hidden += bfloat16(x @ weight.T)`` inside the small-batch product kernel, which also leaves the sums of
    squares of the new ``hidden`` for the next norm.  None when that kernel does not take the sizes: the caller
    then computes the product and hands it to the norm as a pending delta."""
    if not (x.shape[0] <= LAZY_NORM_LIMIT and _takes_small_m(x, weight) and hidden.dtype == torch.float32
            and hidden.is_contiguous() and hidden.shape == (x.shape[0], weight.shape[0])):
        return None
    ssq = torch.empty(((weight.shape[0] + 127) // 128, x.shape[0]), dtype=torch.float32, device=x.device)
    ext().small_m_gemm_residual(x, weight, hidden, ssq, _cluster_splits(weight), status)
    _launched()
    return Summed(hidden, ssq)


def _takes_small_m(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (use_small_m_gemm and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.dim() == 2 and x.shape[0] <= SMALL_M_LIMIT and x.is_contiguous() and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and ext().small_m_gemm_supported(x.shape[0], weight.shape[0], weight.shape[1]))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, partial_ok: bool = False,
           status: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``, float32 accumulation.

    Few bfloat16 tokens (decode steps) go through this package's tcgen05 kernel; everything else is the library
    GEMM, as in the reference.  With ``partial_ok`` the result may be a 3-D float32 stack
    ``[parts, tokens, features]`` of split-K partial sums, for a consumer kernel that adds them up;
    ``out_dtype=torch.float32`` keeps the accumulator's precision in the result (used for the logits).
    ``x`` may be a ``LazyNorm``.
    """
    if isinstance(x, LazyNorm) and bias is not None:
        x = x.materialize()
    x, normed, small = _operand(x, weight)
    if bias is None and small:
        if partial_ok and prefer_partials and not normed:
            return small_m_gemm(x, weight, parts=True, status=status)
        return small_m_gemm(x, weight, out_dtype=out_dtype or torch.bfloat16, status=status, normed=normed)
    if out_dtype is not None and out_dtype != x.dtype:
        out = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            out += bias.to(out_dtype)
        return out
    return torch.nn.functional.linear(x, weight, bias)


# ----------------------------------------------------------------------------- chains of products in one kernel

#: a decode step of at most this many bfloat16 tokens may run the tail of each layer and the head of the next (output
#: projection, gate/up, down, the next q/k/v projection) as ONE persistent kernel that never stops streaming weights
STREAM_LIMIT = 8
#: Off unless AKV_STREAM_PHASES=1: measured on B200 at the benchmark model's sizes the chain of a layer takes 100 us
#: in the persistent kernel against 76 us as four kernels (a decode step of 8 tokens: 4.26 ms against 3.37 ms).  Its
#: weights do stream at the memory's rate (0.37 us per 16 KB block per SM), but each of the three places where a
#: phase needs the one before it finished everywhere costs 5 to 6 us (the last tile's sum over the cluster, a
#: releasing count in global memory, the slowest SM, the operand built anew) against the 3.7 us of weights that the
#: ring holds, and whole tiles per cluster of four leave a share of the SMs idle at the end of each phase (48 tiles
#: over 33 clusters).  Asking the L2 for blocks ahead of the ring made it slower still.
use_stream_phases = os.environ.get("AKV_STREAM_PHASES", "0") == "1"
_STREAM_SYNC_INTS = 1 << 16


class _StreamScratch:
    """Per device: sums of squares, whatever scratch the kernel asks for and its zeroed counters.  The counters
    are handed out slice by slice and zeroed again at the start of every step (``stream_begin_step``)."""

    def __init__(self, device):
        self.device = device
        self.ssq = torch.empty((1,), dtype=torch.float32, device=device)
        self.parts = torch.empty((1,), dtype=torch.float32, device=device)
        self.sync = torch.zeros((_STREAM_SYNC_INTS,), dtype=torch.int32, device=device)
        self.cursor = 0
        self.high_water = 0      # counters ever handed out: a replayed graph may have used them behind our back


_STREAM_SCRATCH: dict = {}


def _device_key(device) -> torch.device:
    """``cuda`` and ``cuda:0`` name the same device: always the form with an index."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def _stream_scratch(device) -> _StreamScratch:
    key = _device_key(device)
    if key not in _STREAM_SCRATCH:
        _STREAM_SCRATCH[key] = _StreamScratch(key)
    return _STREAM_SCRATCH[key]


def stream_begin_step(device) -> None:
    """Zero every counter the chained-product kernel has ever been handed on this device (one small memset; nothing
    before the kernel's first use).  Called at the start of every step, so a captured step carries its own."""
    if not _STREAM_SCRATCH:
        return
    scratch = _STREAM_SCRATCH.get(_device_key(device))
    if scratch is not None and scratch.high_water:
        scratch.sync[:scratch.high_water].zero_()
        scratch.cursor = 0


def stream_phases(hidden: torch.Tensor, phases: list[dict], status: torch.Tensor | None = None,
                  trace: torch.Tensor | None = None) -> None:
    """Run ``phases`` (1 to 4 products, each depending on the one before) on the float32 residual stream ``hidden``
    [tokens <= 16, width] in one persistent kernel.  A phase is a dict: ``w`` [features, k] bfloat16; ``x``
    [tokens, k] bfloat16, or ``norm_weight`` and ``eps`` for the RMS norm of ``hidden``; ``epilogue`` "residual" (adds
    the product, rounded to bfloat16, into ``hidden``), "gated" (``out`` = silu(gate) * up over rows alternating in
    runs of 64), "plain" (``out``) or "qkv" (the arguments of the fused q/k/v projection).  Outputs are written into
    the tensors the phases name."""
    scratch = _stream_scratch(hidden.device)
    part_floats, sync_ints = ext().stream_phases_scratch([(int(p["w"].shape[0]), int(p["w"].shape[1])) for p in phases])
    ssq_floats = (hidden.shape[1] + 127) // 128 * 16
    if scratch.ssq.numel() < ssq_floats:
        scratch.ssq = torch.empty((ssq_floats,), dtype=torch.float32, device=hidden.device)
    if scratch.parts.numel() < part_floats:
        scratch.parts = torch.empty((part_floats,), dtype=torch.float32, device=hidden.device)
    if scratch.cursor + sync_ints > scratch.sync.numel():
        raise RuntimeError("the chained-product kernel ran out of counters: stream_begin_step() was not called "
                           "between steps")
    sync = scratch.sync[scratch.cursor:scratch.cursor + sync_ints]
    scratch.cursor += sync_ints
    scratch.high_water = max(scratch.high_water, scratch.cursor)
    ext().stream_phases(hidden, phases, scratch.ssq, scratch.parts, sync, status, trace)
    _launched()


def stream_takes(tokens: int, *weights: torch.Tensor) -> bool:
    """Whether the chained-product kernel takes a step of ``tokens`` tokens over these matrices."""
    return (use_stream_phases and 1 <= tokens <= STREAM_LIMIT and all(
        w is not None and w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
        and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0 and w.shape[1] >= 64 for w in weights))


class PendingPhases:
    """Products that are decided but not launched yet: the tail of one layer (output projection, feed-forward) waits
    here for the head of the next (its q/k/v projection) so that all of them go into one launch of the
    chained-product kernel.  Whoever needs the residual stream itself calls :meth:`launch` first."""

    def __init__(self, hidden: torch.Tensor, status: torch.Tensor | None = None):
        self.hidden, self.status = hidden, status
        self.phases: list[dict] = []
        self._max = None

    def room(self, count: int = 1) -> bool:
        if self._max is None:
            self._max = int(ext().stream_phases_max())
        return len(self.phases) + count <= self._max

    def add(self, phase: dict) -> None:
        if not self.room():
            self.launch()
        self.phases.append(phase)

    def launch(self) -> None:
        if self.phases:
            stream_phases(self.hidden, self.phases, status=self.status)
            self.phases = []


class StreamNorm:
    """An RMS norm of the residual stream that is not computed: the consumer adds a phase whose token operand the
    chained-product kernel makes from the stream itself, after the phases queued before it."""

    def __init__(self, pending: PendingPhases, weight: torch.Tensor, eps: float, dtype: torch.dtype):
        self.pending, self.weight, self.eps, self.dtype = pending, weight, float(eps), dtype

    @property
    def hidden(self) -> torch.Tensor:
        return self.pending.hidden

    @property
    def shape(self):
        return self.pending.hidden.shape

    def normed_phase(self, w: torch.Tensor, **epilogue) -> dict:
        return dict(w=w, norm_weight=self.weight, eps=self.eps, **epilogue)

    def materialize(self) -> torch.Tensor:
        """Launch what is queued and run the norm kernel after all."""
        self.pending.launch()
        return add_rmsnorm(self.pending.hidden, None, self.weight, self.eps, self.dtype, status=self.pending.status)


# ----------------------------------------------------------------------------- the stream, again

def stream_add(hidden: torch.Tensor, other: torch.Tensor, delta=None):
    """``hidden += other`` in place (both float32 [tokens, width]).  ``delta`` is what a block left pending for the
    stream; what is still pending afterwards is handed back: a plain branch output stays pending, products that are
    queued are launched first, and a record of sums that the stream held before (``Summed``, ``Mirrored``) is
    dropped, since it no longer describes the stream."""
    if isinstance(delta, PendingPhases):
        delta.launch()
        delta = None
    elif isinstance(delta, (Summed, Mirrored)):
        delta = None
    ext().stream_add(hidden, other)
    _launched()
    return delta


def scaled_sum(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float) -> torch.Tensor:
    """``a * sa + b * sb`` of two branch outputs, formed in float32 and rounded once to their dtype."""
    out = torch.empty_like(a)
    ext().scaled_sum(a, b, out, float(sa), float(sb))
    _launched()
    return out


def pair_rows_add(hidden, ids, positions, cu_q, state_slots, last_token, table, *, vocab, buckets, mul_prev, mul_cur,
                  sampled=None) -> torch.Tensor:
    """``hidden[t] += table[(previous token * mul_prev + token * mul_cur) mod buckets]``, and ``table[buckets]`` for a
    token at position 0.  The token before a step's first row is read from ``last_token[slot, 0]`` (int32
    [slots, >= 1]), where the step's last token of every sequence is left for the next step."""
    ext().pair_rows_add(hidden, ids, sampled, positions, cu_q, state_slots, last_token, table, int(vocab), int(buckets),
                        int(mul_prev), int(mul_cur))
    _launched()
    return hidden


# ----------------------------------------------------------------------------- rotary positions before attention

ROTARY_LAYOUTS = {"half": 0, "pairs": 1}


def rotary_prep(x, positions, slots, freq, k_cache, v_cache, *, num_heads, num_kv_heads, head_dim, v_dim, rotary_dims,
                layout: str, factor: float = 1.0, value_from_key: bool = False, value_norm: bool = False,
                eps: float = 0.0, status=None, q_norm=None, k_norm=None, row_norm_eps: float = 0.0,
                x_off: int = 0) -> torch.Tensor:
    """From one product ``x`` [tokens, q heads | k heads (| v heads)]: the first ``rotary_dims`` dims of every q and k
    head turned by ``positions[t] * freq[i]`` (``layout`` ``"half"``: dim i pairs with i + rotary_dims / 2;
    ``"pairs"``: dim 2i with 2i + 1; cos and sin times ``factor``); the value is the v head (divided by its root mean
    square with ``value_norm``), or with ``value_from_key`` the k head before the turn (no v columns then); k and v go
    to their cache slots.  With ``q_norm`` / ``k_norm`` (float32 [heads * head_dim] / [kv heads * head_dim]) the whole q
    row and the whole k row are first divided by their root mean square over all heads (``row_norm_eps`` inside the
    root) and multiplied by these weights.  With ``x_off`` the q, k (and v) columns begin at that column of a wider
    ``x`` (a product shared with another mixer).  Returns q [tokens, heads * head_dim]."""
    q_out = torch.empty((x.shape[0], num_heads * head_dim), dtype=x.dtype, device=x.device)
    ext().rotary_prep(x, positions, slots, freq, q_out, k_cache, v_cache, num_heads, num_kv_heads, head_dim, v_dim,
                      int(rotary_dims), ROTARY_LAYOUTS[layout], float(factor), bool(value_from_key), bool(value_norm),
                      float(eps), status, q_norm, k_norm, float(row_norm_eps), int(x_off))
    _launched()
    return q_out


def rotary_rows(x, positions, freq, *, num_heads, head_dim, v_dim, rotary_dims, q_off: int, k_off: int, v_off: int,
                q_scale: float = 1.0, k_scale: float = 1.0) -> torch.Tensor:
    """The q, k and v heads of one product as float32 rows ``[q | k | v]`` (padded to a multiple of four floats) for a
    scan that keeps everything in float32: the first ``rotary_dims`` dims of every q and k head turned by
    ``positions[t] * freq[i]`` (dim i pairs with i + rotary_dims / 2), then q times ``q_scale`` and k times
    ``k_scale``."""
    width = 2 * num_heads * head_dim + num_heads * v_dim
    out = torch.empty((x.shape[0], (width + 3) // 4 * 4), dtype=torch.float32, device=x.device)
    ext().rotary_rows(x, positions, freq, out, num_heads, head_dim, v_dim, int(rotary_dims), int(q_off), int(k_off),
                      int(v_off), float(q_scale), float(k_scale))
    _launched()
    return out


# ----------------------------------------------------------------------------- linear attention with a decaying memory

LINEAR_SCAN_MAX_DIM = 256
LINEAR_SCAN_MODES = {"gated_write": 0, "constant_decay": 1, "plain_decay": 2, "token_decay": 3}
_SCAN_COLUMNS = 32


def linear_scan_shape(head_dim: int, v_dim: int) -> tuple[int, int] | None:
    """(rows of a value column per lane, lanes per column) of the scan kernel, or None when it does not take the
    sizes."""
    if not (0 < head_dim <= LINEAR_SCAN_MAX_DIM and 0 < v_dim <= LINEAR_SCAN_MAX_DIM):
        return None
    rows, lanes = (16 if head_dim <= 128 else 32), 1
    while lanes * rows < head_dim:
        lanes *= 2
    return (rows, lanes) if lanes <= 8 else None


def linear_scan_state_floats(num_heads: int, head_dim: int, v_dim: int) -> int:
    """Floats of a request's memory (all heads) as the scan kernel lays it out: the key width padded to lanes times
    rows per lane, the value width to slices of 32 columns."""
    rows, lanes = linear_scan_shape(head_dim, v_dim)
    return num_heads * ((v_dim + _SCAN_COLUMNS - 1) // _SCAN_COLUMNS) * _SCAN_COLUMNS * rows * lanes


def linear_scan_memory(state_row: torch.Tensor, num_heads: int, head_dim: int, v_dim: int) -> torch.Tensor:
    """One request's memory ``[heads, head_dim, v_dim]`` read out of its state row (the kernel keeps it in an order of
    its own: [head][slice of 32 columns][row in lane][column][lane])."""
    rows, lanes = linear_scan_shape(head_dim, v_dim)
    slices = (v_dim + _SCAN_COLUMNS - 1) // _SCAN_COLUMNS
    s = state_row[: num_heads * slices * _SCAN_COLUMNS * rows * lanes].view(num_heads, slices, rows, _SCAN_COLUMNS, lanes)
    s = s.permute(0, 4, 2, 1, 3).reshape(num_heads, lanes * rows, slices * _SCAN_COLUMNS)
    return s[:, :head_dim, :v_dim]


def linear_scan(x, state, cu_q, state_slots, *, num_heads, head_dim, v_dim, mode: str, q_off: int, k_off: int,
                v_off: int, gate_bias=None, lower=None, decay=None, qk_group: int = 1, decay_off: int = 0) -> torch.Tensor:
    """``S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t`` per head over the step's tokens, sequence by sequence,
    from and into ``state`` [slots, floats] float32 (:func:`linear_scan_state_floats` of them per slot).  The columns
    of ``x`` from ``q_off`` / ``k_off`` / ``v_off`` hold a product's q, gate-or-key and v.  ``mode`` ``"gated_write"``:
    ``a = f, k = 1 - f`` with ``f = lower + (1 - lower) sigmoid(x_k + gate_bias)``, ``q = silu(x_q)``, ``v = x_v``;
    ``"constant_decay"``: ``a = decay[head]``, q, k and v through SiLU; ``"plain_decay"``: ``a = decay[head]`` and q,
    k, v as they stand in ``x``, which is then float32 (a kernel before has prepared them); ``"token_decay"``: the
    same with ``a = x[t, decay_off + head]``, a scalar per head and token, and ``qk_group`` heads in a row sharing one
    q and one k (the q and k columns then hold ``num_heads / qk_group`` heads).  Returns float32
    [tokens, heads * v_dim]."""
    out = torch.empty((x.shape[0], num_heads * v_dim), dtype=torch.float32, device=x.device)
    ext().linear_scan(x, state, cu_q, state_slots, out, num_heads, head_dim, v_dim, LINEAR_SCAN_MODES[mode], int(q_off),
                      int(k_off), int(v_off), gate_bias, lower, decay, int(qk_group), int(decay_off))
    _launched()
    return out


GATE_KINDS = {"sigmoid": 0, "silu": 1}


def group_norm_gate(o, weight, *, group: int, eps: float, out_dtype, factor: float = 1.0, x=None, gate_off: int = 0,
                    gate: str = "sigmoid", gate_first: bool = False, skip=None, skip_off: int = 0, skip_coef=None,
                    skip_head: int = 1):
    """``v / sqrt(mean over each group of `group` columns of v^2 + eps) * weight * factor`` (``weight`` holds a
    group's or the whole width's entries, or is None), where ``v`` is ``o`` (float32 [tokens, width]), plus
    ``skip_coef[column // skip_head] * skip[:, skip_off + column]`` when ``skip`` (float32) is given.  With ``x`` the
    result is gated by ``sigmoid`` or ``silu`` (``gate``) of ``x[:, gate_off + column]``: after the norm, or with
    ``gate_first`` before it (the gate then enters the root mean square).  The result is in ``out_dtype``."""
    out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    ext().group_norm_gate(o, out, weight, int(group), float(eps), float(factor), x, int(gate_off), GATE_KINDS[gate],
                          bool(gate_first), skip, int(skip_off), skip_coef, int(skip_head))
    _launched()
    return out


# ----------------------------------------------------------------------------- a selective state-space mixer

SSM_MAX_HEADS = 1024
CONV_MAX_TAPS = 16


def ssm_prep_width(num_heads: int, v_dim: int, state_dim: int, groups: int) -> int:
    """Floats of a token's prepared row ``[C | B | dt x | decay | x]``, rounded up to a multiple of four."""
    return (2 * groups * state_dim + 2 * num_heads * v_dim + num_heads + 3) // 4 * 4


def ssm_prep(x, conv, conv_bias, step_bias, rate_log, state, cu_q, state_slots, *, tail_off: int, num_heads, v_dim,
             state_dim, groups, taps, conv_off: int, step_off: int) -> torch.Tensor:
    """From one product ``x`` whose columns from ``conv_off`` hold ``[x (heads * v_dim) | B (groups * state_dim) |
    C (groups * state_dim)]`` and from ``step_off`` a step per head: the channels through their causal convolution
    over the sequence's own earlier tokens (``conv`` float32 [channels, taps], last tap the current token's, plus
    ``conv_bias``; before the step's first token the inputs come from ``state[slot, tail_off:]``) and SiLU;
    ``dt = softplus(step + step_bias)``, ``decay = exp(-exp(rate_log) * dt)``.  Returns float32 rows
    ``[C | B | dt * x | decay | x]``: q, k, v and the per-token decay of ``linear_scan(mode="token_decay")``, and the
    skip input.  The state is not changed."""
    out = torch.empty((x.shape[0], ssm_prep_width(num_heads, v_dim, state_dim, groups)), dtype=torch.float32,
                      device=x.device)
    ext().ssm_prep(x, conv, conv_bias, step_bias, rate_log, state, int(tail_off), cu_q, state_slots, out, num_heads,
                   v_dim, state_dim, groups, taps, int(conv_off), int(step_off))
    _launched()
    return out


def conv_tail(x, state, cu_q, state_slots, *, tail_off: int, conv_off: int, channels: int, taps: int) -> None:
    """Every sequence's last ``taps - 1`` rows of the columns ``[conv_off, conv_off + channels)`` of ``x`` (older rows
    from what the slot held) into ``state[slot, tail_off:]`` as [taps - 1, channels]."""
    if taps <= 1:
        return
    ext().conv_tail(x, state, int(tail_off), cu_q, state_slots, int(conv_off), int(channels), int(taps))
    _launched()


# ----------------------------------------------------------------------------- a residual stream in several copies

HYPER_MAX_STREAMS = 8


class HyperPending:
    """A sublayer's result that is not yet written back into the copies of the stream: ``y`` [tokens, width] with the
    coefficients of its write (``mix`` [streams, streams] from -> to, ``write`` [streams], ``scale`` [width] or None)."""

    def __init__(self, y: torch.Tensor, mix: torch.Tensor, write: torch.Tensor, scale: torch.Tensor | None):
        self.y, self.mix, self.write, self.scale = y, mix, write, scale


def hyper_expand(hidden: torch.Tensor, streams: int) -> torch.Tensor:
    """``streams`` copies of every row: float32 [tokens, width] -> [tokens, streams, width]."""
    x = torch.empty((hidden.shape[0], streams, hidden.shape[1]), dtype=torch.float32, device=hidden.device)
    ext().hyper_expand(hidden, x)
    _launched()
    return x


def hyper_step(x: torch.Tensor, pending: HyperPending | None, read: torch.Tensor | None, weight: torch.Tensor | None,
               eps: float, out_dtype, rows: torch.Tensor | None = None, status=None) -> torch.Tensor | None:
    """One pass over the copies ``x`` [tokens, streams, width] (float32, changed in place): the pending write
    ``x_t <- sum_s mix[s, t] x_s + write[t] * scale * y`` if there is one, then, if ``read`` is given, the next
    sublayer's input ``u = sum_s read[s] x_s`` normed: ``u / sqrt(mean(u^2) + eps) * weight`` in ``out_dtype``
    (only the rows ``rows`` when given; a gather goes without a write)."""
    out = None
    if read is not None:
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, x.shape[2]), dtype=out_dtype, device=x.device)
    if pending is None:
        ext().hyper_step(x, None, None, None, None, read, weight, float(eps), out, rows, status)
    else:
        ext().hyper_step(x, pending.y, pending.mix, pending.write, pending.scale, read, weight, float(eps), out, rows,
                         status)
    _launched()
    return out


def hyper_collapse(x: torch.Tensor, pending: HyperPending | None) -> torch.Tensor:
    """The sum of the copies after the pending write (which is not stored): float32 [tokens, width]."""
    out = torch.empty((x.shape[0], x.shape[2]), dtype=torch.float32, device=x.device)
    if pending is None:
        ext().hyper_collapse(x, None, None, None, None, out)
    else:
        ext().hyper_collapse(x, pending.y, pending.mix, pending.write, pending.scale, out)
    _launched()
    return out


def normed_pair_sum(a, b, wa, wb, *, eps: float, sa: float, sb: float, out_dtype) -> torch.Tensor:
    """``sa * a / sqrt(mean(a^2) + eps) * wa + sb * b / sqrt(mean(b^2) + eps) * wb`` row by row; ``a`` and ``b``
    float32 [tokens, width], the result in ``out_dtype``."""
    out = torch.empty(a.shape, dtype=out_dtype, device=a.device)
    ext().normed_pair_sum(a, b, wa, wb, out, float(eps), float(sa), float(sb))
    _launched()
    return out
