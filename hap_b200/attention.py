"""``F.multi_head_attention_forward`` on a batch shard, through the C ABI.

The planner emits self-attention as one call of
``torch.nn.functional.multi_head_attention_forward(query=x, key=x, value=x, in_proj_weight=...,
in_proj_bias=..., out_proj_weight=..., out_proj_bias=..., attn_mask=..., embed_dim_to_check=E,
num_heads=H, bias_k=None, bias_v=None, add_zero_attn=False, dropout_p=p)`` on (L, N, E) tensors
(``hap.rs:1297-1329``); only N is ever sharded (``hap.rs:2903-2926``).  :func:`multi_head_attention_forward`
takes the same keyword arguments and returns ``(output, None)``; the two projections run on the
package's linear kernels.  The attention core runs as one fused tensor-core kernel per direction for
head dimension 64 (scores, softmax, dropout on the probabilities and the value product stay on the SM;
backward recomputes them), and on batched GEMMs plus softmax kernels for other head dimensions
(without dropout).
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import _native as N
from . import dropout as _dropout
from .comm import _on_device, _stream
from .linear import linear

FUSED_HEAD_DIM = 64


# One program hands the same mask tensor to every layer (the language model builds it once per forward,
# models.py:72): its float32 form and the device word that says "this is just the causal mask" are made
# once per tensor (and per in-place version of it) and reused by all layers, forward and backward.
_mask_cache = {}      # id(mask tensor) -> (weak reference to it, its version, float32 form, flag word)


def _classify_mask(mask: Optional[torch.Tensor], L: int):
    """(causal flag, additive fp32 mask or None, device flag word or None).  A mask tensor is applied as
    an additive (L, L) fp32 term inside the kernels (-inf entries mask, as with the reference's LM mask,
    ``models.py:72``); no value of it is inspected on the host, so nothing synchronises: a small kernel
    leaves a device word that tells the attention kernels whether the tensor is exactly the causal
    mask.  The string ``"causal"`` selects the built-in causal masking without a tensor."""
    if mask is None:
        return 0, None, None
    if isinstance(mask, str):
        if mask != "causal":
            raise ValueError(f"attention: unknown mask {mask!r}")
        return 1, None, None
    hit = _mask_cache.get(id(mask))
    if hit is not None and hit[0]() is mask and hit[1] == mask._version:
        return 0, hit[2], hit[3]
    if mask.dtype == torch.bool:
        add = torch.zeros(mask.shape, dtype=torch.float32, device=mask.device).masked_fill_(mask, float("-inf"))
    else:
        add = mask.float()
    if add.shape != (L, L):
        raise ValueError(f"attention: attn_mask must be ({L}, {L}), got {tuple(add.shape)}")
    add = add.contiguous()
    flag = None
    if add.is_cuda:
        flag = torch.empty(1, dtype=torch.int32, device=add.device)
        with _on_device(add.device):
            N.check(N.lib.hapx_attention_classify_mask(add.data_ptr(), L, flag.data_ptr(), _stream(add.device)))
    key = id(mask)
    _mask_cache[key] = (weakref.ref(mask, lambda _ref, key=key: _mask_cache.pop(key, None)), mask._version, add, flag)
    return 0, add, flag


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, num_heads, causal, mask):
        L, n, e3 = qkv.shape
        E = e3 // 3
        D = E // num_heads
        Lp = (L + 7) // 8 * 8
        qkv = qkv.contiguous()
        out = torch.empty((L, n, E), dtype=torch.bfloat16, device=qkv.device)
        probs = torch.empty((n * num_heads, L, Lp), dtype=torch.bfloat16, device=qkv.device)
        scores = torch.empty((n * num_heads, L, Lp), dtype=torch.float32, device=qkv.device)
        with _on_device(qkv.device):
            N.check(N.lib.hapx_attention_forward(out.data_ptr(), probs.data_ptr(), scores.data_ptr(), qkv.data_ptr(), L, n,
                                                 num_heads, D, int(causal), mask.data_ptr() if mask is not None else None,
                                                 _stream(qkv.device)))
        ctx.save_for_backward(qkv, probs)
        ctx.meta = (L, n, num_heads, D)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, probs = ctx.saved_tensors
        L, n, H, D = ctx.meta
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dscores = torch.empty(probs.shape, dtype=torch.float32, device=qkv.device)
        ds = torch.empty_like(probs)
        with _on_device(qkv.device):
            N.check(N.lib.hapx_attention_backward(dqkv.data_ptr(), dscores.data_ptr(), ds.data_ptr(), dout.data_ptr(),
                                                  probs.data_ptr(), qkv.data_ptr(), L, n, H, D, _stream(qkv.device)))
        return dqkv, None, None, None


class _FusedAttention(torch.autograd.Function):
    """The fused kernels (head dimension 64): saves qkv, the output and one float per row."""

    @staticmethod
    def forward(ctx, qkv, num_heads, causal, mask, mask_flag, dropout_p, call_id):
        L, n, e3 = qkv.shape
        E = e3 // 3
        qkv = qkv.contiguous()
        out = torch.empty((L, n, E), dtype=torch.bfloat16, device=qkv.device)
        lse2 = torch.empty((n * num_heads, L), dtype=torch.float32, device=qkv.device)
        with _on_device(qkv.device):
            N.check(N.lib.hapx_attention_fused_forward(out.data_ptr(), lse2.data_ptr(), qkv.data_ptr(), L, n, num_heads, FUSED_HEAD_DIM,
                                                       int(causal), mask.data_ptr() if mask is not None else None,
                                                       mask_flag.data_ptr() if mask_flag is not None else None, float(dropout_p),
                                                       int(call_id), _stream(qkv.device)))
        ctx.save_for_backward(qkv, out, lse2, mask, mask_flag)
        ctx.meta = (L, n, num_heads, int(causal), float(dropout_p), int(call_id))
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse2, mask, mask_flag = ctx.saved_tensors
        L, n, H, causal, dropout_p, call_id = ctx.meta
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty_like(lse2)
        with _on_device(qkv.device):
            N.check(N.lib.hapx_attention_fused_backward(dqkv.data_ptr(), delta.data_ptr(), dout.data_ptr(), out.data_ptr(), lse2.data_ptr(),
                                                        qkv.data_ptr(), L, n, H, FUSED_HEAD_DIM, causal,
                                                        mask.data_ptr() if mask is not None else None,
                                                        mask_flag.data_ptr() if mask_flag is not None else None, dropout_p, call_id,
                                                        _stream(qkv.device)))
        return dqkv, None, None, None, None, None, None


def attention_keep_mask(L: int, n: int, num_heads: int, dropout_p: float, call_id: int, device=None) -> torch.Tensor:
    """The keep mask (uint8, (n * num_heads, L, L)) the fused kernels draw for attention call ``call_id``
    in the current iteration."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    mask = torch.empty((n * num_heads, L, L), dtype=torch.uint8, device=device)
    with _on_device(device):
        N.check(N.lib.hapx_attention_dropout_mask(mask.data_ptr(), L, n, num_heads, float(dropout_p), int(call_id), _stream(device)))
    return mask


def attention(qkv: torch.Tensor, num_heads: int, attn_mask: Optional[torch.Tensor] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """softmax(Q K^T / sqrt(d) + mask) V for packed ``qkv`` of shape (L, N, 3E), bfloat16, on CUDA, with
    dropout on the probabilities when ``dropout_p`` > 0."""
    if not qkv.is_cuda:
        raise RuntimeError(f"attention: hap_b200 has no CPU path; tensor is on {qkv.device}")
    if qkv.dtype != torch.bfloat16:
        raise TypeError(f"attention: bfloat16 only, got {qkv.dtype}")
    if qkv.dim() != 3 or qkv.shape[2] % (3 * num_heads):
        raise ValueError("attention: qkv must be (L, N, 3 * num_heads * head_dim)")
    causal, mask, mask_flag = _classify_mask(attn_mask, qkv.shape[0])
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError(f"attention: dropout_p must be in [0, 1), got {dropout_p}")
    if qkv.shape[2] // (3 * num_heads) == FUSED_HEAD_DIM and qkv.shape[1] > 0:
        call_id = _dropout.new_call_id() if dropout_p > 0.0 else 0
        return _FusedAttention.apply(qkv, num_heads, causal, mask, mask_flag, dropout_p, call_id)
    if dropout_p > 0.0:
        raise NotImplementedError("attention: dropout on the probabilities needs head dimension 64 (the fused kernels)")
    return _Attention.apply(qkv, num_heads, causal, mask)


def multi_head_attention_forward(query, key, value, embed_dim_to_check, num_heads, in_proj_weight, in_proj_bias,
                                 bias_k=None, bias_v=None, add_zero_attn=False, dropout_p=0.0, out_proj_weight=None,
                                 out_proj_bias=None, training=True, key_padding_mask=None, need_weights=True, attn_mask=None,
                                 use_separate_proj_weight=False, **unsupported):
    """Same call surface as ``torch.nn.functional.multi_head_attention_forward`` for the case the planner
    emits (self-attention, packed projection).  Returns ``(attn_output, None)``."""
    if not (query is key and key is value):
        raise NotImplementedError("attention: only self-attention (query is key is value) is emitted by the planner")
    if bias_k is not None or bias_v is not None or add_zero_attn or key_padding_mask is not None or use_separate_proj_weight:
        raise NotImplementedError("attention: bias_k / bias_v / add_zero_attn / key_padding_mask / separate weights are not emitted by the planner")
    if query.shape[-1] != embed_dim_to_check:
        raise ValueError("attention: embedding dimension mismatch")
    qkv = linear(query, in_proj_weight, in_proj_bias)
    out = attention(qkv, num_heads, attn_mask, float(dropout_p) if training else 0.0)
    return linear(out, out_proj_weight, out_proj_bias), None
